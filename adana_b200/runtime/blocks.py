"""Manual forward and backward of a dense pre-norm transformer block, the embedding and the
loss head, written over the functional ops of `adana_b200.ops`.

One generic block covers both architectures:
  Enoki : LayerNorm, fused c_attn (q|k|v), per-head QK-LayerNorm + RoPE, GELU MLP
  Qwen3 : RMSNorm (or LayerNorm), fused [q(+gate)|k|v] projection, per-head QK-norm + RoPE,
          optional sigmoid output gate, SwiGLU MLP, grouped-query attention
The residual stream (and its gradient) is fp32; every GEMM operand is in the compute dtype
(bf16 on a GPU).  Each GEMM carries the elementwise work next to it in its epilogue:
    qkv   = ln1 · Wqkvᵀ                              bf16
    x_mid = x + s · (attn ⊙ gate) · Woᵀ              fp32 residual epilogue
    z,h   = gelu-dual(ln2 · Wfcᵀ) | gu,h = swiglu(ln2 · Wguᵀ)
    x_out = x_mid + s · h · Wdownᵀ                   fp32 residual epilogue
and in backward  dz = (dy·Wdown) ⊙ act'(z)  is one dgrad GEMM, weight gradients accumulate
straight into the fp32 flat gradient buffer (beta = 1 after the first micro-step), and the
norm backward adds into the residual gradient in place while emitting its bf16 copy for the
next GEMM.

The same code runs on CPU through the PyTorch reference implementation of every op, which is
how the backward formulas are tested against autograd.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..ops import attention as A
from ..ops import gemm as G
from ..ops import misc as M
from ..ops import norm as N
from ..ops import rope as R


@dataclass
class BlockSpec:
    d: int
    n_head: int
    n_kv_head: int
    hd: int
    mlp: int
    mlp_kind: str            # "gelu" | "swiglu"
    norm_kind: int           # block norms: 0 LayerNorm, 1 RMSNorm
    qk_kind: int             # per-head norm: 0 LN, 1 RMS, 2 none
    gate: bool               # sigmoid output gate packed into the q projection
    eps: float
    qk_eps: float
    scale: float             # residual_stream_scalar
    seq_len: int

    # column layout of the fused projection output
    @property
    def q_hstride(self):
        return 2 * self.hd if self.gate else self.hd

    @property
    def nq(self):
        return self.n_head * self.q_hstride

    @property
    def nkv(self):
        return self.n_kv_head * self.hd

    @property
    def k_off(self):
        return self.nq

    @property
    def v_off(self):
        return self.nq + self.nkv

    @property
    def proj_out(self):
        return self.nq + 2 * self.nkv


def _row_parallel_resid(tp, a, w, resid, alpha):
    """resid + alpha * sum over tp ranks of a_r · w_rᵀ (each rank holds a slice of the contraction)."""
    M, N = a.shape[0], w.shape[0]

    def produce(out):
        if out is None:
            return (a.float() @ w.float().t()) * alpha
        return G.gemm(a, w, out, M=M, N=N, K=a.shape[1], alpha=alpha)

    return tp.sum_partials(produce, M, N, resid=resid)


def _col_parallel_dgrad(tp, dy, w):
    """sum over tp ranks of dy_r · w_r: the input gradient of a column-parallel linear."""
    M, K = dy.shape[0], w.shape[1]

    def produce(out):
        if out is None:
            return dy.float() @ w.float()
        return G.linear_dgrad(dy, w, out=out)

    return tp.sum_partials(produce, M, K)


def block_forward(x, W: Dict[str, torch.Tensor], sp: BlockSpec, freqs, B: int, S: int, cdt,
                  need_grad: bool = True, tp=None):
    """x fp32 [T, d] -> (x_out fp32 [T, d], saved dict or None).  With `tp` (a TensorParallelGroup) the weights are this
    rank's slices, `sp` counts its heads and hidden units, and the two row-parallel products are summed over tp."""
    ln1, mean1, rstd1 = N.norm_fwd(x, W["ln_1"], sp.eps, sp.norm_kind, cdt)
    qkv = G.linear_fwd(ln1, W["qkv"])
    q, k = R.qknorm_rope_fwd(qkv, 0, sp.q_hstride, sp.k_off, sp.hd, W.get("q_norm"), W.get("k_norm"),
                             freqs, S, sp.n_head, sp.n_kv_head, sp.hd, sp.qk_eps, sp.qk_kind)
    y, actx = A.attention_fwd(q, k, qkv, sp.v_off, sp.hd, B, S, need_grad=need_grad)
    yg = M.sigmoid_gate_fwd(y, qkv, sp.hd, sp.q_hstride, sp.n_head, sp.hd) if sp.gate else y
    x_mid = G.linear_resid_fwd(yg, W["o"], x, alpha=sp.scale) if tp is None else _row_parallel_resid(tp, yg, W["o"], x, sp.scale)
    ln2, mean2, rstd2 = N.norm_fwd(x_mid, W["ln_2"], sp.eps, sp.norm_kind, cdt)
    if sp.mlp_kind == "gelu":
        z, h = G.linear_gelu_fwd(ln2, W["fc"])
    else:
        z, h = G.linear_swiglu_fwd(ln2, W["fc"])
    x_out = (G.linear_resid_fwd(h, W["down"], x_mid, alpha=sp.scale) if tp is None
             else _row_parallel_resid(tp, h, W["down"], x_mid, sp.scale))
    if not need_grad:
        return x_out, None
    saved = dict(x=x, ln1=ln1, mean1=mean1, rstd1=rstd1, qkv=qkv, q=q, k=k, y=y, yg=yg, actx=actx,
                 x_mid=x_mid, ln2=ln2, mean2=mean2, rstd2=rstd2, z=z, h=h)
    return x_out, saved


def block_backward(dx, dx_lp, sv, W, Gd: Dict[str, torch.Tensor], sp: BlockSpec, freqs, B: int, S: int,
                   acc: bool, tp=None):
    """dx (fp32, grad w.r.t. the block output) is updated in place to the grad w.r.t. the block
    input; dx_lp is its compute-dtype copy (also updated).  Weight grads go to `Gd` (fp32 views),
    accumulated when `acc` else overwritten."""
    s = sp.scale
    # ---- MLP branch ----
    if sp.mlp_kind == "gelu":
        dz = G.linear_dgrad_dgelu(dx_lp, W["down"], sv["z"], alpha=s)
    else:
        dz = G.linear_dgrad_dswiglu(dx_lp, W["down"], sv["z"], alpha=s)
    G.linear_wgrad(dx_lp, sv["h"], out=Gd["down"], accumulate=acc, alpha=s)
    G.linear_wgrad(dz, sv["ln2"], out=Gd["fc"], accumulate=acc)
    dln2 = G.linear_dgrad(dz, W["fc"]) if tp is None else _col_parallel_dgrad(tp, dz, W["fc"])
    del dz
    N.norm_bwd(dln2, sv["x_mid"], W["ln_2"], sv["mean2"], sv["rstd2"], sp.norm_kind, dx_accum=dx,
               dw_out=Gd["ln_2"], dw_accumulate=acc, dx_lowp=dx_lp)
    del dln2
    # ---- attention branch ----
    dyg = G.linear_dgrad(dx_lp, W["o"], alpha=s)
    G.linear_wgrad(dx_lp, sv["yg"], out=Gd["o"], accumulate=acc, alpha=s)
    qkv = sv["qkv"]
    dqkv = torch.empty_like(qkv)
    if sp.gate:
        dy = M.sigmoid_gate_bwd(dyg, sv["y"], qkv, dqkv, sp.hd, sp.q_hstride, sp.n_head, sp.hd)
    else:
        dy = dyg
    dq, dk = A.attention_bwd(dy, sv["q"], sv["k"], qkv, sp.v_off, sp.hd, B, S, sv["actx"], dqkv)
    fold = tp is None and "q_norm" in Gd        # (under tensor parallelism the two gradients are first summed over tp)
    dwq, dwk = R.qknorm_rope_bwd(dq, dk, qkv, dqkv, 0, sp.q_hstride, sp.k_off, sp.hd, W.get("q_norm"),
                                 W.get("k_norm"), freqs, S, sp.n_head, sp.n_kv_head, sp.hd, sp.qk_eps,
                                 sp.qk_kind, dw_out=(Gd["q_norm"], Gd["k_norm"]) if fold else None, dw_accumulate=acc)
    if dwq is not None and not fold:
        if tp is not None:          # the per-head norm weights are shared by all heads: their gradient sums over tp
            both = tp.all_reduce_(torch.cat([dwq.reshape(-1), dwk.reshape(-1)]))
            dwq, dwk = both[:dwq.numel()].view_as(dwq), both[dwq.numel():].view_as(dwk)
        for key, val in (("q_norm", dwq), ("k_norm", dwk)):
            if acc:
                Gd[key] += val
            else:
                Gd[key].copy_(val)
    del dq, dk, dy, dyg
    G.linear_wgrad(dqkv, sv["ln1"], out=Gd["qkv"], accumulate=acc)
    dln1 = G.linear_dgrad(dqkv, W["qkv"]) if tp is None else _col_parallel_dgrad(tp, dqkv, W["qkv"])
    del dqkv
    N.norm_bwd(dln1, sv["x"], W["ln_1"], sv["mean1"], sv["rstd1"], sp.norm_kind, dx_accum=dx,
               dw_out=Gd["ln_1"], dw_accumulate=acc, dx_lowp=dx_lp)
    return dx, dx_lp


def head_forward_backward(x, targets, W, Gd, sp_norm_kind: int, eps: float, z_coeff: float,
                          loss_scale: float, cdt, need_grad: bool, acc: bool):
    """Final norm + LM head + CE/z-loss (+ accuracy).  When `need_grad`, also returns the fp32
    gradient w.r.t. x (and its compute-dtype copy) and accumulates dW of lm_head / ln_f."""
    T, d = x.shape
    xf, mean, rstd = N.norm_fwd(x, W["ln_f"], eps, sp_norm_kind, cdt)
    if targets is None:
        # labels drawn from the model's own distribution, a chunk of logits at a time
        targets = torch.empty(T, dtype=torch.long, device=x.device)
        with torch.no_grad():
            for s0 in range(0, T, 4096):
                logits = G.linear_fwd(xf[s0:s0 + 4096], W["lm_head"]).float()
                targets[s0:s0 + 4096] = torch.distributions.Categorical(logits=logits).sample()
    if need_grad and not acc:
        Gd["lm_head"].zero_()
    res = M.linear_ce(xf, W["lm_head"], targets.reshape(-1), z_coeff, loss_scale, need_grad=need_grad,
                      dw_out=Gd["lm_head"] if need_grad else None)
    ce = res["ce_sum"] / T
    z = res["z_sum"] / T
    out = {"ce": ce, "z": z, "loss": ce + z_coeff * z, "correct": res["correct"], "valid": res["valid"]}
    if not need_grad:
        return out, None, None
    dx_lp = torch.empty((T, d), dtype=cdt, device=x.device)
    dx, _ = N.norm_bwd(res["dh"], x, W["ln_f"], mean, rstd, sp_norm_kind, dx_accum=None,
                       dw_out=Gd["ln_f"], dw_accumulate=acc, dx_lowp=dx_lp)
    return out, dx, dx_lp


def hoyer_value_and_grad(x0: torch.Tensor, coeff: float, loss_scale: float, need_grad: bool):
    """Hoyer sparsity term on the token embeddings: mean ||x||_1 / (||x||_2 + 1e-8)."""
    if not need_grad:
        # two row reductions that read x0 once each and write one float per token (no |x| temporary)
        l1 = torch.linalg.vector_norm(x0, ord=1, dim=-1)
        return (l1 / (torch.linalg.vector_norm(x0, ord=2, dim=-1) + 1e-8)).mean(), None
    xd = x0.detach().requires_grad_(True)
    with torch.enable_grad():
        val = (xd.abs().sum(-1) / (xd.norm(dim=-1) + 1e-8)).mean()
        g, = torch.autograd.grad(val * (coeff * loss_scale), xd)
    return val.detach(), g
