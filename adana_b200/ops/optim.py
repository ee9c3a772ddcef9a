"""Fused flat-shard optimizer step and gradient-norm helpers (csrc/optim.cu).

`FlatOptimizerState` holds fp32 (p, m, v[, tau]) for one flat shard and applies the ADana-family
or AdamW update in one kernel, also writing the bf16 copy of the parameters.  On CPU the same
math runs through `adana_b200.optim.logtime.logtime_update_`.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ..optim.logtime import logtime_update_

KIND_ADANA, KIND_DANA_STAR, KIND_ADAMW, KIND_ADAMW_IWD, KIND_ADEMAMIX, KIND_ADEMAMIX_IWD = 0, 1, 2, 3, 4, 5


def cast_f32_to_bf16(src: torch.Tensor, dst: torch.Tensor):
    """dst (bf16) = round(src (fp32)), one pass (the wire copy of a gradient unit)."""
    if src.is_cuda and _lib.available() and src.is_contiguous() and dst.is_contiguous():
        rc = _lib.lib().adana_cast_f32_to_bf16(src.data_ptr(), dst.data_ptr(), src.numel(), _lib.stream_ptr())
        _lib.check_rc(rc, "adana_cast_f32_to_bf16")
    else:
        dst.copy_(src)
    return dst


def sumsq_accumulate(x: torch.Tensor, out: torch.Tensor):
    """out[0] += sum(x^2) (fp32)."""
    if x.is_cuda and _lib.available() and x.dtype == torch.float32 and x.is_contiguous():
        rc = _lib.lib().adana_sumsq_f32(x.data_ptr(), x.numel(), out.data_ptr(), _lib.stream_ptr())
        _lib.check_rc(rc, "adana_sumsq_f32")
    else:
        out[0] += x.float().pow(2).sum()
    return out


def clip_coef(sumsq: torch.Tensor, norm_scale: float, max_norm: float, out: torch.Tensor):
    """out[0] = min(1, max_norm/(norm+1e-6)) (1 when max_norm == 0), out[1] = norm = sqrt(sumsq)*norm_scale."""
    if sumsq.is_cuda and _lib.available():
        rc = _lib.lib().adana_clip_coef(sumsq.data_ptr(), float(norm_scale), float(max_norm), out.data_ptr(),
                                        _lib.stream_ptr())
        _lib.check_rc(rc, "adana_clip_coef")
    else:
        norm = sumsq[0].sqrt() * norm_scale
        out[1] = norm
        out[0] = torch.clamp(max_norm / (norm + 1e-6), max=1.0) if max_norm > 0 else 1.0
    return out


def make_hyper(*, kind, lr, alpha, step, kappa, clipsnr, eps, gamma3, wd_factor, grad_scale=1.0, betas=(0.9, 0.999),
               beta3=0.0, wd_coupled=0.0):
    """The C struct of per-launch optimizer scalars."""
    h = _lib.AdanaOptHyper()
    h.lr, h.alpha, h.step = float(lr), float(alpha), float(step)
    h.one_minus_kappa = float(1.0 - kappa)
    h.clipsnr = -1.0 if clipsnr is None else float(clipsnr)
    h.eps, h.gamma3, h.wd_factor, h.grad_scale = float(eps), float(gamma3), float(wd_factor), float(grad_scale)
    h.kind = int(kind)
    b1, b2 = betas
    h.beta1, h.beta2 = float(b1), float(b2)
    h.bc1, h.bc2 = float(1 - b1 ** step), float(1 - b2 ** step)
    h.beta3, h.wd_coupled = float(beta3), float(wd_coupled)
    return h


def fused_step(p, g, m, v, tau, p16, *, kind, lr, alpha, step, kappa, clipsnr, eps, gamma3, wd_factor,
               grad_scale=1.0, clip_coef_t=None, betas=(0.9, 0.999), diag=None, beta3=0.0, wd_coupled=0.0):
    """One fused update of a flat fp32 range.  All tensors are 1-D and contiguous."""
    n = p.numel()
    if n == 0:
        return
    if p.is_cuda and _lib.available():
        h = make_hyper(kind=kind, lr=lr, alpha=alpha, step=step, kappa=kappa, clipsnr=clipsnr, eps=eps, gamma3=gamma3,
                       wd_factor=wd_factor, grad_scale=grad_scale, betas=betas, beta3=beta3, wd_coupled=wd_coupled)
        rc = _lib.lib().adana_opt_step(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), _lib.ptr(tau),
                                       _lib.ptr(p16), n, ctypes.byref(h), _lib.ptr(clip_coef_t), _lib.ptr(diag),
                                       _lib.stream_ptr())
        _lib.check_rc(rc, "adana_opt_step")
        return
    # reference path (CPU): same math through the PyTorch formulation
    gs = g * grad_scale
    if clip_coef_t is not None:
        gs = gs * clip_coef_t[0]
    if kind in (KIND_ADANA, KIND_DANA_STAR):
        d = logtime_update_(p, gs, m, v, tau if kind == KIND_DANA_STAR else None, lr=lr, alpha=alpha, step=step,
                            kappa=kappa, clipsnr=clipsnr, eps=eps, gamma3=gamma3, wd_mult=wd_factor,
                            diagnostics=diag is not None)
        if diag is not None:
            nel = float(n)
            diag[0] += d["current_alpha"] * nel
            diag[1] += d["gradient_norm"] ** 2
            diag[2] += d["auto_factor_mean"] * nel
            diag[3] += d["m_norm"] ** 2
    elif kind in (KIND_ADEMAMIX, KIND_ADEMAMIX_IWD):
        b1, b2 = betas
        m.mul_(b1).add_(gs, alpha=1 - b1)
        tau.mul_(beta3).add_(gs, alpha=1 - beta3)
        v.mul_(b2).addcmul_(gs, gs, value=1 - b2)
        denom = (v.sqrt() / (1 - b2 ** step) ** 0.5).add_(eps)
        upd = (m / (1 - b1 ** step) + alpha * gamma3 * tau) / denom
        if kind == KIND_ADEMAMIX_IWD:
            p.mul_(wd_factor)
        else:
            upd.add_(p, alpha=wd_coupled)
        p.add_(upd, alpha=-lr)
    else:
        b1, b2 = betas
        if kind == KIND_ADAMW:
            p.mul_(wd_factor)
        m.mul_(b1).add_(gs, alpha=1 - b1)
        v.mul_(b2).addcmul_(gs, gs, value=1 - b2)
        denom = (v.sqrt() / (1 - b2 ** step) ** 0.5).add_(eps)
        p.addcdiv_(m, denom, value=-lr / (1 - b1 ** step))
        if kind == KIND_ADAMW_IWD:
            p.mul_(wd_factor)
    if p16 is not None:
        p16.copy_(p)
