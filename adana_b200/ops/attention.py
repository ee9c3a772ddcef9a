"""Causal self-attention forward / backward (and forward-mode tangent) entry points.

`attention_fwd` / `attention_bwd` take q [T, Hq, hd], k [T, Hk, hd] (contiguous, from the
QK-norm+RoPE kernel) and v as a strided view into the fused projection output, with T = B*S.
Grouped-query attention (Hk < Hq) maps query head h to KV head h // (Hq/Hk).

Implementations, in order of preference on a GPU:
  1. the hand-written tcgen05/TMA kernels of csrc/attention_tcgen05.cu (when built in and the
     shape is supported);
  2. PyTorch SDPA (library kernel) — the interim path and the comparator in benchmarks.
The CPU reference is a plain fp32 masked softmax.  Replaces F.scaled_dot_product_attention of
the reference (src/models/enoki.py:134-136, src/models/qwen3.py:212-217).
"""
from __future__ import annotations

import math
import os

import torch
import torch.nn.functional as F

from . import _lib

# auto | native | sdpa | ref.  "auto" resolves to the hand-written tcgen05 kernels whenever they cover the
# shape (bf16, head_dim 64 or 128, sequence length a multiple of 128) and to the library kernel otherwise.
# cuDNN's kernels are still faster in isolation (see benchmarks/attention_bench.py): `set_mode("sdpa")` /
# ADANA_ATTENTION=sdpa / --attention sdpa selects them.
_FORCE = os.environ.get("ADANA_ATTENTION", "auto")


def set_mode(mode: str) -> None:
    global _FORCE
    assert mode in ("auto", "native", "sdpa", "ref")
    _FORCE = mode


def get_mode() -> str:
    return _FORCE


def _v_view(vbuf, v_off, v_hstride, Hk, hd):
    T = vbuf.shape[0]
    return torch.as_strided(vbuf, (T, Hk, hd), (vbuf.stride(0), v_hstride, 1), vbuf.storage_offset() + v_off)


def native_supported(q, hd, S) -> bool:
    return (q.is_cuda and _lib.available() and _lib.has("adana_attn_fwd") and q.dtype == torch.bfloat16
            and hd in (64, 128) and S % 128 == 0)


def attention_ref(q, k, v, B, S, scale):
    """fp32 reference: q [T,Hq,hd], k/v [T,Hk,hd] -> out [T, Hq*hd], lse [B,Hq,S]."""
    T, Hq, hd = q.shape
    Hk = k.shape[1]
    qf = q.float().view(B, S, Hq, hd).transpose(1, 2)
    kf = k.float().view(B, S, Hk, hd).transpose(1, 2).repeat_interleave(Hq // Hk, dim=1)
    vf = v.float().reshape(B, S, Hk, hd).transpose(1, 2).repeat_interleave(Hq // Hk, dim=1)
    s = (qf @ kf.transpose(-1, -2)) * scale
    mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.softmax(s, -1) @ vf
    return o.transpose(1, 2).reshape(T, Hq * hd), lse


def attention_fwd(q, k, vbuf, v_off, v_hstride, B, S, scale=None, need_grad=True):
    """Returns (out [T, Hq*hd] in q.dtype, ctx) where ctx carries what backward needs."""
    T, Hq, hd = q.shape
    Hk = k.shape[1]
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    v = _v_view(vbuf, v_off, v_hstride, Hk, hd)
    mode = _FORCE
    if mode == "auto":
        mode = "native" if native_supported(q, hd, S) else ("sdpa" if q.is_cuda else "ref")
    if mode == "native" and not native_supported(q, hd, S):
        mode = "sdpa" if q.is_cuda else "ref"
    if mode == "native":
        from . import attention_native

        if need_grad and not attention_native.bwd_available():
            mode = "sdpa"   # no native backward built in: keep forward and backward on one implementation
        else:
            out, lse = attention_native.fwd(q, k, vbuf, v_off, v_hstride, B, S, scale)
            return out, ("native", lse, out)
    if mode == "sdpa":
        # library kernel; the autograd graph of this one call is kept for the backward sweep
        qd, kd, vd = (t.detach().requires_grad_(need_grad) for t in (q, k, v))
        with torch.set_grad_enabled(need_grad):
            o = F.scaled_dot_product_attention(
                qd.view(B, S, Hq, hd).transpose(1, 2), kd.view(B, S, Hk, hd).transpose(1, 2),
                torch.as_strided(vd, (B, Hk, S, hd), (S * vd.stride(0), vd.stride(1), vd.stride(0), 1),
                                 vd.storage_offset()),
                is_causal=True, scale=scale, enable_gqa=(Hk != Hq))
            out = o.transpose(1, 2).reshape(T, Hq * hd)
        return out.detach(), ("sdpa", (qd, kd, vd, out) if need_grad else None, None)
    if need_grad:
        qd, kd, vd = (t.detach().requires_grad_(True) for t in (q, k, v))
        with torch.enable_grad():
            out, lse = attention_ref(qd, kd, vd, B, S, scale)
        return out.detach().to(q.dtype), ("ref", (qd, kd, vd, out), None)
    out, lse = attention_ref(q, k, v, B, S, scale)
    return out.to(q.dtype), ("ref", None, None)


def attention_bwd(dout, q, k, vbuf, v_off, v_hstride, B, S, ctx, dvbuf, scale=None):
    """Returns (dq [T,Hq,hd], dk [T,Hk,hd]); writes dv into `dvbuf` (projection layout)."""
    T, Hq, hd = q.shape
    Hk = k.shape[1]
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    mode = ctx[0]
    if mode == "native":
        from . import attention_native

        return attention_native.bwd(dout, q, k, vbuf, v_off, v_hstride, B, S, scale, ctx[1], ctx[2], dvbuf)
    qd, kd, vd, o = ctx[1]
    dq, dk, dv = torch.autograd.grad(o, [qd, kd, vd], dout.to(o.dtype))
    _v_view(dvbuf, v_off, v_hstride, Hk, hd).copy_(dv.to(dvbuf.dtype))
    return dq.to(q.dtype), dk.to(k.dtype)
