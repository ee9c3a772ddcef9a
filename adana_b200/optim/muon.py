"""Muon-type optimizers: Newton–Schulz orthogonalised momentum for weight matrices.

* `newton_schulz5`      quintic iteration (a,b,c) = (3.4445, -4.7750, 2.0315); X <- aX + (bA + cA²)X with
                        A = XXᵀ, in bf16, on the wide orientation (reference src/optim/muon.py:19-47).
                        On a GPU the three GEMMs of an iteration run on the tcgen05 kernels
                        (`adana_b200.ops.muon_ns`); the PyTorch form below is the oracle.
* `Muon`                rank-partitioned Muon for replicated (DDP) parameters: parameter i is
                        orthogonalised by rank i mod N, results are exchanged with one bf16 all-reduce
                        (reference src/optim/muon.py:443-602).
* `DistributedMuon`     Moonlight-style Muon (lr scaled by 0.2*sqrt(max(A,B)), decoupled WD) with AdamW
                        for vectors, embeddings and the head (reference src/optim/muon.py:126-440).  Under
                        the sharded engine the gather → NS → scatter chain of
                        `adana_b200/parallel/dist_muon.py` is used instead of per-matmul redistributes.
* `Manau`               Muon on block matrices + Dana-Star-MK4 elsewhere (reference src/optim/manau.py:89-601).
* `CombinedScheduler`   one LR scheduler per parameter group for `--opt muon`
                        (reference src/optim/muon.py:660-752); `cos` maps to a cosine with floor
                        1/final_div_factor, which the reference names but does not define.
"""
from __future__ import annotations

import math
import os

import torch
import torch.distributed as dist
from torch.optim import Optimizer

from .schedule import CosInf, WSD

NS_COEFFS = (3.4445, -4.7750, 2.0315)


def newton_schulz5(G: torch.Tensor, steps: int = 5, eps: float = 1e-7, dtype=None) -> torch.Tensor:
    """Approximate orthogonal factor of a 2-D matrix (singular values pushed towards 1)."""
    assert G.dim() == 2
    a, b, c = NS_COEFFS
    X = G if dtype is None else G.to(dtype)
    tall = G.size(0) > G.size(1)
    if tall:
        X = X.T
    X = X / (X.norm() + eps)
    for _ in range(steps):
        A = X @ X.T
        B = b * A + c * (A @ A)
        X = a * X + B @ X
    return X.T if tall else X


zeropower_via_newtonschulz5 = newton_schulz5  # the reference's name


def orthogonalize(G: torch.Tensor, steps: int) -> torch.Tensor:
    """Dispatch: tcgen05 chain on a GPU, PyTorch oracle elsewhere."""
    if G.is_cuda:
        from adana_b200.ops import muon_ns

        if muon_ns.supported(G):
            return muon_ns.newton_schulz5_cuda(G, steps)
    return newton_schulz5(G, steps)


def adjust_lr_for_muon(lr: float, matched_adamw_rms: float, shape) -> float:
    A, B = shape[:2]
    return lr * math.sqrt(max(A, B)) * matched_adamw_rms


def _adamw_like_step(p, g, state, k1, k2, step, lr, wd, betas, eps):
    """The Muon codebases' AdamW: lerp moments, eps inside the raw sqrt, joint bias scale."""
    b1, b2 = betas
    if k1 not in state:
        state[k1] = torch.zeros_like(g)
        state[k2] = torch.zeros_like(g)
    state[k1].lerp_(g, 1 - b1)
    state[k2].lerp_(g.square(), 1 - b2)
    upd = state[k1] / (eps + state[k2].sqrt())
    scale = (1 - b1 ** step) / (1 - b2 ** step) ** 0.5
    p.mul_(1 - lr * wd)
    p.add_(upd, alpha=-lr / scale)


class Muon(Optimizer):
    def __init__(self, muon_params, lr=0.02, momentum=0.95, nesterov=True, ns_steps=6,
                 adamw_params=None, adamw_lr=3e-4, adamw_betas=(0.95, 0.95), adamw_eps=1e-8,
                 adamw_wd=0):
        defaults = dict(lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps,
                        adamw_lr=adamw_lr, adamw_lr_ratio=adamw_lr / lr, adamw_betas=adamw_betas,
                        adamw_eps=adamw_eps, adamw_wd=adamw_wd)
        muon_params = list(muon_params)
        adamw_params = list(adamw_params) if adamw_params is not None else []
        super().__init__(muon_params + adamw_params, defaults)
        for p in muon_params:
            self.state[p]["use_muon"] = p.ndim >= 2 and p.size(0) < 10000
        for p in adamw_params:
            self.state[p]["use_muon"] = False
        if dist.is_available() and dist.is_initialized():
            self.world_size, self.rank = dist.get_world_size(), dist.get_rank()
        else:
            self.world_size, self.rank = 1, 0

    @torch.no_grad()
    def step(self, closure=None):
        for group in self.param_groups:
            mats = [p for p in group["params"] if self.state[p]["use_muon"]]
            lr, mu = group["lr"], group["momentum"]
            if mats:
                flat = torch.zeros(sum(p.numel() for p in mats), device=mats[0].device,
                                   dtype=torch.bfloat16)
                off = 0
                for i, p in enumerate(mats):
                    if i % self.world_size == self.rank:
                        g = p.grad.reshape(p.grad.size(0), -1)
                        st = self.state[p]
                        if "momentum_buffer" not in st:
                            st["momentum_buffer"] = torch.zeros_like(g)
                        buf = st["momentum_buffer"].mul_(mu).add_(g)
                        upd = g.add(buf, alpha=mu) if group["nesterov"] else buf
                        upd = orthogonalize(upd.to(torch.bfloat16), group["ns_steps"])
                        upd = upd * max(1, upd.size(0) / upd.size(1)) ** 0.5
                        flat[off:off + p.numel()] = upd.flatten()
                    off += p.numel()
                if self.world_size > 1:
                    dist.all_reduce(flat, op=dist.ReduceOp.SUM)
                off = 0
                for p in mats:
                    p.add_(flat[off:off + p.numel()].view_as(p).to(p.dtype), alpha=-lr)
                    off += p.numel()
            lr_a = group["adamw_lr_ratio"] * group["lr"]
            for p in group["params"]:
                if self.state[p]["use_muon"] or p.grad is None:
                    continue
                st = self.state[p]
                st["step"] = st.get("step", 0) + 1
                _adamw_like_step(p, p.grad, st, "moment1", "moment2", st["step"], lr_a,
                                 group["adamw_wd"], group["adamw_betas"], group["adamw_eps"])


class DistributedMuon(Optimizer):
    def __init__(self, param_groups, lr=2e-2, weight_decay=0.1, matched_adamw_rms=0.2, momentum=0.95,
                 nesterov=True, ns_steps=5, adamw_betas=(0.95, 0.95), adamw_eps=1e-8):
        defaults = dict(lr=lr, weight_decay=weight_decay, matched_adamw_rms=matched_adamw_rms,
                        momentum=momentum, nesterov=nesterov, ns_steps=ns_steps,
                        adamw_betas=adamw_betas, adamw_eps=adamw_eps)
        super().__init__(param_groups, defaults)
        self.distributed_mode = False
        for group in self.param_groups:
            for p in group["params"]:
                self.state[p]["use_muon"] = p.ndim >= 2 and p.size(0) < 10000

    @torch.no_grad()
    def step(self, closure=None):
        for group in self.param_groups:
            lr, wd, mu = group["lr"], group["weight_decay"], group["momentum"]
            group["step"] = group.get("step", 0) + 1
            for p in group["params"]:
                g = p.grad
                if g is None:
                    continue
                st = self.state[p]
                if st.get("use_muon", False):
                    if "muon_buffer" not in st:
                        st["muon_buffer"] = torch.zeros_like(g)
                    buf = st["muon_buffer"].mul_(mu).add_(g)
                    ns_in = (g.add(buf, alpha=mu) if group["nesterov"] else buf).to(torch.bfloat16)
                    upd = orthogonalize(ns_in, group["ns_steps"])
                    p.mul_(1 - lr * wd)
                    p.add_(upd.to(p.dtype), alpha=-adjust_lr_for_muon(lr, group["matched_adamw_rms"], ns_in.shape))
                else:
                    _adamw_like_step(p, g, st, "adamw_exp_avg", "adamw_exp_avg_sq", group["step"], lr,
                                     wd, group["adamw_betas"], group["adamw_eps"])


class Manau(Optimizer):
    _NON_MATRIX_NAMES = ("wte.weight", "wpe.weight", "lm_head.weight")

    def __init__(self, param_groups, lr=2e-2, weight_decay=0.1, matched_adamw_rms=0.2, momentum=0.95,
                 nesterov=True, ns_steps=5, dana_momentum=False, delta=8.0, kappa=1.0, mk4A=0.0,
                 mk4B=0.0, clipsnr=1.0, epsilon=1e-8, weight_time=False, wd_decaying=False, wd_ts=1.0,
                 verbose=False):
        defaults = dict(lr=lr, weight_decay=weight_decay, matched_adamw_rms=matched_adamw_rms,
                        momentum=momentum, nesterov=nesterov, ns_steps=ns_steps,
                        dana_momentum=dana_momentum, delta=delta, kappa=kappa, mk4A=mk4A, mk4B=mk4B,
                        clipsnr=clipsnr, epsilon=epsilon, weight_time=weight_time,
                        wd_decaying=wd_decaying, wd_ts=wd_ts, weighted_step_count=0)
        super().__init__(param_groups, defaults)
        self.lr = lr
        self.distributed_mode = False
        n_muon = n_dana = 0
        for group in self.param_groups:
            names = group.get("param_names")
            if names is None:
                raise ValueError("Manau optimizer requires 'param_names' to be provided in param_groups.")
            for name, p in zip(names, group["params"]):
                emb_or_head = any(tag in name for tag in self._NON_MATRIX_NAMES)
                use = (not emb_or_head) and p.ndim >= 2
                self.state[p]["use_muon"] = use
                if use:
                    n_muon += p.numel()
                else:
                    n_dana += p.numel()
        if verbose:
            tot = max(1, n_muon + n_dana)
            print(f"[Manau] Muon params {n_muon:,} ({100 * n_muon / tot:.1f}%), "
                  f"Dana-Star-MK4 params {n_dana:,} ({100 * n_dana / tot:.1f}%)")

    @staticmethod
    def _tau_reg(tau, step):
        ct = tau.clamp(max=0.5)
        return torch.maximum(ct / (1.0 - ct), torch.full_like(tau, 1.0 / (1.0 + step)))

    @torch.no_grad()
    def step(self, closure=None):
        for group in self.param_groups:
            lr, wd = group["lr"], group["weight_decay"]
            delta, kappa, eps = group["delta"], group["kappa"], group["epsilon"]
            weight_time = group["weight_time"]
            for p in group["params"]:
                g = p.grad
                if g is None:
                    continue
                st = self.state[p]
                tf = lr / self.lr if weight_time else 1.0
                if st.get("use_muon", False):
                    if "muon_buffer" not in st:
                        st["muon_buffer"] = torch.zeros_like(g)
                        st["step"] = 0
                    st["step"] += 1
                    buf = st["muon_buffer"]
                    if group["dana_momentum"]:
                        group["weighted_step_count"] += tf
                        t = group["weighted_step_count"] if weight_time else st["step"]
                        alpha = delta / (delta + t) * tf
                        buf.mul_(1 - alpha).add_(g, alpha=alpha)
                        ns_in = g + buf * st["step"] ** (1 - kappa)
                    else:
                        buf.mul_(group["momentum"]).add_(g)
                        ns_in = g.add(buf, alpha=group["momentum"]) if group["nesterov"] else buf
                    ns_in = ns_in.to(torch.bfloat16)
                    upd = orthogonalize(ns_in, group["ns_steps"])
                    p.mul_(1 - lr * wd)
                    p.add_(upd.to(p.dtype), alpha=-adjust_lr_for_muon(lr, group["matched_adamw_rms"], ns_in.shape))
                    continue
                if "dana_m" not in st:
                    st["dana_m"] = torch.zeros_like(g)
                    st["dana_v"] = torch.zeros_like(g)
                    st["dana_tau"] = torch.zeros_like(g)
                    st["step"] = 0
                m, v, tau = st["dana_m"], st["dana_v"], st["dana_tau"]
                st["step"] += 1
                group["weighted_step_count"] += tf
                t = group["weighted_step_count"] if weight_time else st["step"]
                alpha = delta / (delta + t) * tf
                m.mul_(1 - alpha).add_(g, alpha=alpha)
                v.mul_(1 - alpha).addcmul_(g, g, value=alpha)
                ag = g.abs()
                tau.mul_(1 - alpha).add_(ag / (ag + v.sqrt() + eps), alpha=alpha)
                reg = self._tau_reg(tau, t)
                eff_t = torch.maximum(tau * t, torch.ones_like(tau))
                norm = reg.sqrt() / (v.sqrt() + eps)
                mfac = norm * m.abs() / reg
                af = torch.clamp(eff_t ** (1 - kappa) * mfac ** (2 * group["mk4B"] + 1)
                                 * norm ** (2 * (-group["mk4A"] - group["mk4B"])), max=group["clipsnr"])
                long_term = lr * (reg * torch.sign(m) * af + m * norm)
                st["current_alpha"] = alpha
                st["current_alpha_factor"] = af.mean().full_tensor() if hasattr(af, "full_tensor") else af.mean()
                full = lambda v: v.full_tensor() if hasattr(v, "full_tensor") else v      # (reduced, so the state can be saved)
                st["gradient_norm"] = full(g.norm())
                st["auto_factor_mean"] = full(mfac.mean())
                st["m_norm"] = full(m.norm())
                if wd != 0:
                    p.mul_(1 - wd / (1 + t / group["wd_ts"]) * lr if group["wd_decaying"] else 1 - wd * lr)
                p.add_(-(lr * g * norm + long_term))


class CombinedScheduler:
    """Applies the configured schedule shape to every parameter group of a Muon optimizer."""

    def __init__(self, optimizer, cfg, muon_lr_key="lr", adamw_lr_key="adamw_lr"):
        self.schedulers = []
        LambdaLR = torch.optim.lr_scheduler.LambdaLR
        shapes = {
            "cos": lambda: CosInf(cfg.iterations, cfg.warmup_steps, 1e2, cfg.final_div_factor, 0),
            "cos_inf": lambda: CosInf(cfg.iterations, cfg.warmup_steps, cfg.div_factor,
                                      cfg.final_div_factor, cfg.cos_inf_steps),
            "wsd": lambda: WSD(cfg.iterations, cfg.wsd_final_lr_scale, cfg.warmup_steps, 1e2,
                               cfg.wsd_fract_decay, cfg.decay_type),
        }
        for group in optimizer.param_groups:
            key = muon_lr_key if muon_lr_key in group else adamw_lr_key
            if key not in group:
                continue
            if cfg.scheduler == "linear":
                s = torch.optim.lr_scheduler.OneCycleLR(
                    optimizer, max_lr=[g.get(key, cfg.lr) for g in optimizer.param_groups],
                    total_steps=cfg.iterations, pct_start=cfg.warmup_steps / cfg.iterations,
                    anneal_strategy="linear", cycle_momentum=False, div_factor=1e2, final_div_factor=1)
            elif cfg.scheduler in shapes:
                s = LambdaLR(optimizer, shapes[cfg.scheduler]())
            else:
                continue
            self.schedulers.append(s)
            if cfg.scheduler == "linear":
                break  # OneCycleLR already carries every group's peak rate
            # otherwise one (identical, idempotent) LambdaLR per parameter group, as the reference keeps them
            # (src/optim/muon.py:718-738): its checkpoints hold `scheduler_0 .. scheduler_{G-1}`

    def step(self):
        for s in self.schedulers:
            s.step()

    def get_last_lr(self):
        return self.schedulers[0].get_last_lr() if self.schedulers else []

    def state_dict(self):
        return {f"scheduler_{i}": s.state_dict() for i, s in enumerate(self.schedulers)}

    def load_state_dict(self, sd):
        for i, s in enumerate(self.schedulers):
            s.load_state_dict(sd[f"scheduler_{i}"])
