"""LayerNorm (weight only) / RMSNorm forward and backward (csrc/norm.cu) with PyTorch references.

Functional, no autograd: the block engine calls `norm_fwd` in the forward sweep and `norm_bwd`
in the backward sweep.  `kind`: 0 = LayerNorm (mean-subtracting, no bias), 1 = RMSNorm.
"""
from __future__ import annotations

import torch

from . import _lib

LAYERNORM, RMSNORM = 0, 1
_PARTIAL_ROWS = 148 * 3   # CTAs of the backward kernel: three of 256 threads fit an SM at cols <= 3072 ...
_PARTIAL_ROWS_192 = 148 * 4   # ... four of the 192-thread variant that rows of 768, 1536 or 2304 columns take
_MAX_COLS = 8192


def _cuda_ok(x, cols):
    return x.is_cuda and _lib.available() and cols % 4 == 0 and cols <= _MAX_COLS


def norm_fwd_ref(x, w, eps, kind, out_dtype):
    xf = x.float()
    if kind == LAYERNORM:
        mean = xf.mean(-1, keepdim=True)
        var = ((xf - mean) ** 2).mean(-1, keepdim=True)
    else:
        mean = torch.zeros_like(xf[..., :1])
        var = (xf * xf).mean(-1, keepdim=True)
    rstd = torch.rsqrt(var + eps)
    y = ((xf - mean) * rstd * w.float()).to(out_dtype)
    return y, mean.squeeze(-1), rstd.squeeze(-1)


def norm_fwd(x, w, eps=1e-5, kind=LAYERNORM, out_dtype=torch.bfloat16):
    """x [rows, cols] (fp32 or bf16) -> (y, mean, rstd)."""
    rows, cols = x.shape
    if not _cuda_ok(x, cols) or out_dtype not in (torch.bfloat16, torch.float32) \
            or x.dtype not in (torch.bfloat16, torch.float32) \
            or (x.dtype == torch.bfloat16 and out_dtype == torch.float32):
        return norm_fwd_ref(x, w, eps, kind, out_dtype)
    x = x.contiguous()
    y = torch.empty((rows, cols), dtype=out_dtype, device=x.device)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    rc = _lib.lib().adana_norm_fwd(x.data_ptr(), int(x.dtype == torch.bfloat16), w.data_ptr(),
                                   y.data_ptr(), int(out_dtype == torch.bfloat16), mean.data_ptr(),
                                   rstd.data_ptr(), rows, cols, float(eps), int(kind), _lib.stream_ptr())
    _lib.check_rc(rc, "adana_norm_fwd")
    return y, mean, rstd


def norm_bwd_ref(dy, x, w, mean, rstd, kind, dx_accum=None):
    xf, dyf = x.float(), dy.float()
    xh = (xf - mean[:, None]) * rstd[:, None]
    g = dyf * w.float()
    m2 = (g * xh).mean(-1, keepdim=True)
    m1 = g.mean(-1, keepdim=True) if kind == LAYERNORM else 0.0
    dx = rstd[:, None] * (g - m1 - xh * m2)
    dw = (dyf * xh).sum(0)
    if dx_accum is not None:
        dx_accum += dx
        dx = dx_accum
    return dx, dw


def norm_bwd(dy, x, w, mean, rstd, kind=LAYERNORM, dx_accum=None, dw_out=None, dw_accumulate=False,
             dx_lowp=None):
    """Returns (dx fp32, dw fp32).  `dx_accum` (fp32, same shape) is added to in place;
    `dx_lowp` (same shape, compute dtype) receives a low-precision copy of the final dx."""
    rows, cols = x.shape
    if not _cuda_ok(x, cols) or dy.dtype not in (torch.bfloat16, torch.float32) \
            or (dy.dtype == torch.float32 and x.dtype == torch.bfloat16):
        dx, dw = norm_bwd_ref(dy, x, w, mean, rstd, kind, dx_accum)
        if dw_out is not None:
            if dw_accumulate:
                dw_out += dw
            else:
                dw_out.copy_(dw)
            dw = dw_out
        if dx_lowp is not None:
            dx_lowp.copy_(dx)
        return dx, dw
    dy = dy.contiguous()
    x = x.contiguous()
    dx = dx_accum if dx_accum is not None else torch.empty((rows, cols), dtype=torch.float32, device=x.device)
    nparts = min(_PARTIAL_ROWS_192 if cols in (768, 1536, 2304) else _PARTIAL_ROWS, rows)
    partial = torch.empty((nparts, cols), dtype=torch.float32, device=x.device)
    lib = _lib.lib()
    rc = lib.adana_norm_bwd(dy.data_ptr(), int(dy.dtype == torch.bfloat16), x.data_ptr(),
                            int(x.dtype == torch.bfloat16), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                            dx.data_ptr(), int(dx_accum is not None), partial.data_ptr(), nparts,
                            rows, cols, int(kind),
                            _lib.ptr(dx_lowp) if (dx_lowp is not None and dx_lowp.dtype == torch.bfloat16) else 0,
                            _lib.stream_ptr())
    _lib.check_rc(rc, "adana_norm_bwd")
    if dx_lowp is not None and dx_lowp.dtype != torch.bfloat16:
        dx_lowp.copy_(dx)
    if dw_out is None:
        dw_out = torch.empty(cols, dtype=torch.float32, device=x.device)
        dw_accumulate = False
    rc = lib.adana_colsum_f32(partial.data_ptr(), nparts, cols, dw_out.data_ptr(), int(dw_accumulate),
                              _lib.stream_ptr())
    _lib.check_rc(rc, "adana_colsum_f32")
    return dx, dw_out
