"""Python side of the hand-written tcgen05 attention kernels (csrc/attention_tcgen05.cu).

`fwd` returns the attention output [T, Hq*hd] (bf16) and `lse2` [B, Hq, S]: the row-wise
log-sum-exp of the scaled scores in log2 units.  `bwd` consumes them.
"""
from __future__ import annotations

import torch

from . import _lib


def fwd(q, k, vbuf, v_off, v_hstride, B, S, scale):
    T, Hq, hd = q.shape
    Hk = k.shape[1]
    out = torch.empty((T, Hq * hd), dtype=torch.bfloat16, device=q.device)
    lse2 = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device)
    vbase = vbuf.data_ptr() + 2 * v_off
    rc = _lib.lib().adana_attn_fwd(q.data_ptr(), k.data_ptr(), vbase, vbuf.stride(0), v_hstride, out.data_ptr(),
                                   lse2.data_ptr(), B, S, Hq, Hk, hd, float(scale),
                                   _lib.status_buffer(q.device).data_ptr(), _lib.stream_ptr())
    _lib.check_rc(rc, "adana_attn_fwd")
    return out, lse2


def bwd_available() -> bool:
    return _lib.has("adana_attn_bwd")


def bwd(dout, q, k, vbuf, v_off, v_hstride, B, S, scale, lse2, out, dvbuf):
    """Returns (dq [T,Hq,hd] fp32, dk [T,Hk,hd] bf16) and writes dv into `dvbuf` at the projection's v columns.  dq is
    the fp32 buffer the kernel's TMA reduce-adds accumulated into; the QK-norm + RoPE backward reads it as it is."""
    T, Hq, hd = q.shape
    Hk = k.shape[1]
    dq_acc = torch.empty((T, Hq, hd), dtype=torch.float32, device=q.device)      # cleared by the delta pass of the kernel call
    dk = torch.empty((T, Hk, hd), dtype=torch.bfloat16, device=q.device)
    delta = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device)
    vbase = vbuf.data_ptr() + 2 * v_off
    dvbase = dvbuf.data_ptr() + 2 * v_off
    rc = _lib.lib().adana_attn_bwd(dout.data_ptr(), q.data_ptr(), k.data_ptr(), vbuf.stride(0), v_hstride, vbase,
                                   out.data_ptr(), lse2.data_ptr(), delta.data_ptr(), dq_acc.data_ptr(),
                                   dk.data_ptr(), dvbuf.stride(0), v_hstride, dvbase, B, S, Hq, Hk, hd,
                                   float(scale), _lib.status_buffer(q.device).data_ptr(), _lib.stream_ptr())
    _lib.check_rc(rc, "adana_attn_bwd")
    return dq_acc, dk


# ---- forward-mode derivative ------------------------------------------------------------------------------------
def jvp_available() -> bool:
    return _lib.available() and _lib.has("adana_attn_jvp")


def jvp(q, k, v, tq, tk, tv, B, S, scale=None):
    """Causal attention and its directional derivative in one kernel (csrc/attention_jvp_tcgen05.cu).

    q, tq [T, Hq, hd]; k, tk, v, tv [T, Hk, hd]; contiguous bf16; returns (out, tangent_out), each [T, Hq*hd]."""
    T, Hq, hd = q.shape
    Hk = k.shape[1]
    scale = hd ** -0.5 if scale is None else scale
    for t in (q, k, v, tq, tk, tv):
        if t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise ValueError("attention jvp takes contiguous bf16 tensors")
    out = torch.empty((T, Hq * hd), dtype=torch.bfloat16, device=q.device)
    tout = torch.empty_like(out)
    rc = _lib.lib().adana_attn_jvp(q.data_ptr(), tq.data_ptr(), k.data_ptr(), tk.data_ptr(), v.data_ptr(),
                                   tv.data_ptr(), out.data_ptr(), tout.data_ptr(), B, S, Hq, Hk, hd, float(scale),
                                   _lib.status_buffer(q.device).data_ptr(), _lib.stream_ptr())
    _lib.check_rc(rc, "adana_attn_jvp")
    return out, tout


def jvp_ref(q, k, v, tq, tk, tv, B, S, scale=None):
    """fp32 oracle: torch.func.jvp through a plain PyTorch causal attention of the same layout."""
    from .attention import attention_ref

    hd = q.shape[-1]
    scale = hd ** -0.5 if scale is None else scale

    def f(q_, k_, v_):
        return attention_ref(q_, k_, v_, B, S, scale)[0]

    prim = tuple(t.float() for t in (q, k, v))
    tang = tuple(t.float() for t in (tq, tk, tv))
    return torch.func.jvp(f, prim, tang)
