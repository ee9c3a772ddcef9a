"""Per-head QK-norm + rotary embedding, forward and backward (csrc/rope.cu), with references.

The q and k vectors are read in place from the fused projection output `qkv` ([tokens, row]):
q of head h starts at column `q_off + h*q_hstride`, k at `k_off + h*k_hstride`.  Outputs are
contiguous [tokens, heads, hd] bf16 tensors (compute dtype on the reference path).
`freqs` is the [S, hd/2, 2] fp32 (cos, sin) table; token t has position t % S.
"""
from __future__ import annotations

import torch

from . import _lib

LAYERNORM, RMSNORM, NONORM = 0, 1, 2
_PARTIAL = 148 * 2      # CTAs of the backward kernel (two of its 128-register CTAs fit an SM) = partial weight-gradient rows


def precompute_freqs_cis(dim: int, end: int, theta: float = 10000.0) -> torch.Tensor:
    """[end, dim/2, 2] table of (cos, sin) of pos * theta^(-2i/dim) in fp32."""
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2)[: dim // 2].float() / dim))
    ang = torch.outer(torch.arange(end).float(), inv)
    return torch.stack((torch.cos(ang), torch.sin(ang)), dim=-1)


def _gather_heads(qkv, off, hstride, H, hd):
    T = qkv.shape[0]
    return torch.as_strided(qkv, (T, H, hd), (qkv.stride(0), hstride, 1), qkv.storage_offset() + off)


def _norm_ref(x, w, eps, kind):
    if kind == NONORM:
        return x
    if kind == LAYERNORM:
        mean = x.mean(-1, keepdim=True)
        var = ((x - mean) ** 2).mean(-1, keepdim=True)
        return (x - mean) * torch.rsqrt(var + eps) * w
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w


def _rope_ref(x, freqs, S):
    T, H, hd = x.shape
    pos = torch.arange(T, device=x.device) % S
    f = freqs.to(x.device)[pos]                    # [T, hd/2, 2]
    xr = x.reshape(T, H, hd // 2, 2)
    c, s = f[:, None, :, 0], f[:, None, :, 1]
    o0 = xr[..., 0] * c - xr[..., 1] * s
    o1 = xr[..., 0] * s + xr[..., 1] * c
    return torch.stack((o0, o1), dim=-1).reshape(T, H, hd)


def qknorm_rope_fwd_ref(qkv, q_off, q_hstride, k_off, k_hstride, wq, wk, freqs, S, Hq, Hk, hd, eps, kind):
    q = _gather_heads(qkv, q_off, q_hstride, Hq, hd).float()
    k = _gather_heads(qkv, k_off, k_hstride, Hk, hd).float()
    q = _rope_ref(_norm_ref(q, None if wq is None else wq.float(), eps, kind), freqs, S)
    k = _rope_ref(_norm_ref(k, None if wk is None else wk.float(), eps, kind), freqs, S)
    return q.to(qkv.dtype), k.to(qkv.dtype)


def qknorm_rope_fwd(qkv, q_off, q_hstride, k_off, k_hstride, wq, wk, freqs, S, Hq, Hk, hd, eps=1e-5,
                    kind=LAYERNORM):
    T = qkv.shape[0]
    if not (qkv.is_cuda and _lib.available() and qkv.dtype == torch.bfloat16 and hd in (64, 128)):
        return qknorm_rope_fwd_ref(qkv, q_off, q_hstride, k_off, k_hstride, wq, wk, freqs, S, Hq, Hk,
                                   hd, eps, kind)
    q = torch.empty((T, Hq, hd), dtype=torch.bfloat16, device=qkv.device)
    k = torch.empty((T, Hk, hd), dtype=torch.bfloat16, device=qkv.device)
    rc = _lib.lib().adana_qknorm_rope_fwd(
        qkv.data_ptr(), qkv.stride(0), q_off, q_hstride, k_off, k_hstride, _lib.ptr(wq), _lib.ptr(wk),
        freqs.data_ptr(), q.data_ptr(), k.data_ptr(), T, S, Hq, Hk, hd, float(eps), int(kind),
        _lib.stream_ptr())
    _lib.check_rc(rc, "adana_qknorm_rope_fwd")
    return q, k


def qknorm_rope_bwd_ref(dq, dk, qkv, dqkv, q_off, q_hstride, k_off, k_hstride, wq, wk, freqs, S, Hq, Hk,
                        hd, eps, kind):
    outs = []
    for d, off, hs, H, w in ((dq, q_off, q_hstride, Hq, wq), (dk, k_off, k_hstride, Hk, wk)):
        x = _gather_heads(qkv, off, hs, H, hd).float().detach().requires_grad_(True)
        wf = None if w is None else w.float().detach().requires_grad_(True)
        with torch.enable_grad():
            y = _rope_ref(_norm_ref(x, wf, eps, kind), freqs, S)
        ins = [x] + ([wf] if (wf is not None and kind != NONORM) else [])
        grads = torch.autograd.grad(y, ins, d.float())
        _gather_heads(dqkv, off, hs, H, hd).copy_(grads[0].to(dqkv.dtype))
        outs.append(grads[1] if len(grads) > 1 else None)
    return outs[0], outs[1]


def qknorm_rope_bwd(dq, dk, qkv, dqkv, q_off, q_hstride, k_off, k_hstride, wq, wk, freqs, S, Hq, Hk, hd,
                    eps=1e-5, kind=LAYERNORM, dw_out=None, dw_accumulate=False):
    """Writes dq/dk (in the projection layout) into `dqkv`; returns (dwq, dwk) fp32 or None.  `dq` may be fp32 (the
    attention backward's accumulator as it is) or bf16; `dk` is bf16.  With `dw_out = (dwq, dwk)` (fp32 [hd] each) the
    weight gradients are folded straight into those buffers (added when `dw_accumulate`) and are what is returned."""
    T = qkv.shape[0]
    if not (qkv.is_cuda and _lib.available() and qkv.dtype == torch.bfloat16 and hd in (64, 128)):
        dwq, dwk = qknorm_rope_bwd_ref(dq, dk, qkv, dqkv, q_off, q_hstride, k_off, k_hstride, wq, wk, freqs,
                                       S, Hq, Hk, hd, eps, kind)
        if dw_out is not None and dwq is not None:
            for val, out in ((dwq, dw_out[0]), (dwk, dw_out[1])):
                if dw_accumulate:
                    out += val
                else:
                    out.copy_(val)
            return dw_out
        return dwq, dwk
    assert dqkv.stride(0) == qkv.stride(0)
    lib = _lib.lib()
    if kind != NONORM:
        pq = torch.empty((_PARTIAL, hd), dtype=torch.float32, device=qkv.device)
        pk = torch.empty((_PARTIAL, hd), dtype=torch.float32, device=qkv.device)
    else:
        pq = pk = None
    rc = lib.adana_qknorm_rope_bwd(
        dq.data_ptr(), dk.data_ptr(), qkv.data_ptr(), qkv.stride(0), q_off, q_hstride, k_off, k_hstride,
        _lib.ptr(wq), _lib.ptr(wk), freqs.data_ptr(), dqkv.data_ptr(), _lib.ptr(pq), _lib.ptr(pk),
        _PARTIAL, T, S, Hq, Hk, hd, float(eps), int(kind), int(dq.dtype == torch.float32), _lib.stream_ptr())
    _lib.check_rc(rc, "adana_qknorm_rope_bwd")
    if kind == NONORM:
        return None, None
    if dw_out is not None:
        # the deterministic column-sum kernel of the norm backward folds the per-CTA partial rows
        for part, out in ((pq, dw_out[0]), (pk, dw_out[1])):
            _lib.check_rc(lib.adana_colsum_f32(part.data_ptr(), _PARTIAL, hd, out.data_ptr(), int(dw_accumulate),
                                               _lib.stream_ptr()), "adana_colsum_f32")
        return dw_out
    return pq.sum(0), pk.sum(0)
