"""Embedding gather/scatter, fused linear + cross-entropy (+ z-loss, accuracy) and the sigmoid
output gate.  Functional forward/backward pairs with PyTorch references for CPU.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib, gemm


def _cuda(*ts):
    return all(t is None or t.is_cuda for t in ts) and _lib.available()


# ---- embedding ------------------------------------------------------------------------------------
def embedding_fwd(idx, table):
    """idx [T] int64, table [V, d] (fp32 or bf16) -> fp32 [T, d] (the residual stream)."""
    T = idx.numel()
    V, d = table.shape
    if not _cuda(idx, table) or d % 4 or table.dtype not in (torch.float32, torch.bfloat16):
        return table[idx.reshape(-1)].float()
    out = torch.empty((T, d), dtype=torch.float32, device=table.device)
    rc = _lib.lib().adana_embedding_fwd(idx.data_ptr(), table.data_ptr(), int(table.dtype == torch.bfloat16),
                                        out.data_ptr(), T, d, V, _lib.stream_ptr())
    _lib.check_rc(rc, "adana_embedding_fwd")
    return out


def embedding_bwd(idx, dout, dtable):
    """dtable [V, d] fp32 += scatter of dout [T, d] fp32 rows."""
    T = idx.numel()
    V, d = dtable.shape
    if not _cuda(idx, dout, dtable) or d % 4 or dout.dtype != torch.float32:
        dtable.index_add_(0, idx.reshape(-1), dout.to(dtable.dtype))
        return dtable
    rc = _lib.lib().adana_embedding_bwd(idx.data_ptr(), dout.contiguous().data_ptr(), dtable.data_ptr(), T, d, V,
                                        _lib.stream_ptr())
    _lib.check_rc(rc, "adana_embedding_bwd")
    return dtable


# ---- fused linear cross-entropy ---------------------------------------------------------------------
def linear_ce_ref(h, w, targets, z_coeff, loss_scale, need_grad=True, dw_out=None):
    """Reference: full logits in fp32.  Returns dict(ce_sum, z_sum, correct, valid, dh, dw)."""
    hf = h.float().detach().requires_grad_(need_grad)
    wf = w.float().detach().requires_grad_(need_grad)
    T = h.shape[0]
    with torch.enable_grad():
        logits = hf @ wf.t()
        lse = torch.logsumexp(logits, -1)
        ce_sum = F.cross_entropy(logits, targets, ignore_index=-1, reduction="sum")
        z_sum = (lse ** 2).sum()
        total = (ce_sum + z_coeff * z_sum) / T
    out = {"ce_sum": ce_sum.detach(), "z_sum": z_sum.detach(),
           "correct": (logits.argmax(-1) == targets).sum().float(),
           "valid": (targets >= 0).sum().float(), "dh": None, "dw": None}
    if need_grad:
        dh, dw = torch.autograd.grad(total * loss_scale, [hf, wf])
        out["dh"] = dh
        if dw_out is not None:
            dw_out += dw.to(dw_out.dtype)
            dw = dw_out
        out["dw"] = dw
    return out


def linear_ce(h, w, targets, z_coeff=0.0, loss_scale=1.0, need_grad=True, dw_out=None, chunk_rows=8192,
              logits_dtype=torch.bfloat16):
    """lm_head GEMM + CE + z-loss + accuracy, forward AND backward in one sweep over row chunks.

    h [T, d] bf16, w [V, d] bf16, targets [T] int64 (-1 = ignore).  Logits exist only one chunk at a time.  With
    `logits_dtype` bf16 (the default; the reference's autocast also hands bf16 logits to its fp32 cross-entropy,
    src/models/chunked_loss.py:68-151) the tcgen05 GEMM writes the chunk in bf16 and the CE kernel turns it into
    dlogits IN PLACE; with fp32 the GEMM writes fp32 logits and the CE kernel writes a separate bf16 dlogits chunk.
    dlogits feed the dgrad GEMM (dh) and the accumulating wgrad GEMM (dw).  loss = (ce_sum + z_coeff*z_sum) / T and
    the returned gradients are those of `loss_scale * loss`.  8192-row chunks measured best at V = 50304, d = 2304
    (8.6 ms per 16384 tokens against 9.9 ms with 4096 rows, where the fp32 weight gradient is re-read twice as often,
    and 9.5 ms with one 16384-row chunk).
    """
    T, d = h.shape
    V = w.shape[0]
    if not (_cuda(h, w, targets) and h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and V % 8 == 0):
        return linear_ce_ref(h, w, targets, z_coeff, loss_scale, need_grad, dw_out)
    dev = h.device
    lib = _lib.lib()
    sums = torch.zeros(4, dtype=torch.float32, device=dev)
    chunk_rows = min(chunk_rows, T)
    in_place = logits_dtype == torch.bfloat16 and _lib.has("adana_ce_fwd_bwd_bf16")
    if in_place:
        logits = torch.empty((chunk_rows, V), dtype=torch.bfloat16, device=dev)
        dlogits = logits if need_grad else None
    else:
        logits = torch.empty((chunk_rows, V), dtype=torch.float32, device=dev)
        dlogits = torch.empty((chunk_rows, V), dtype=torch.bfloat16, device=dev) if need_grad else None
    dh = torch.empty((T, d), dtype=torch.bfloat16, device=dev) if need_grad else None
    dw = None
    if need_grad:
        dw = dw_out if dw_out is not None else torch.zeros((V, d), dtype=torch.float32, device=dev)
    gscale = float(loss_scale) / T
    for s in range(0, T, chunk_rows):
        e = min(T, s + chunk_rows)
        n = e - s
        hc = h[s:e]
        if in_place:
            gemm.linear_fwd(hc, w, out=logits[:n])
            rc = lib.adana_ce_fwd_bwd_bf16(logits.data_ptr(), V, targets[s:e].data_ptr(), n, V, float(z_coeff), gscale,
                                           _lib.ptr(dlogits), V, sums.data_ptr(), 0, _lib.stream_ptr())
        else:
            gemm.linear_fwd_f32(hc, w, out=logits[:n])
            rc = lib.adana_ce_fwd_bwd(logits.data_ptr(), V, targets[s:e].data_ptr(), n, V, float(z_coeff), gscale,
                                      _lib.ptr(dlogits), V, sums.data_ptr(), 0, _lib.stream_ptr())
        _lib.check_rc(rc, "adana_ce_fwd_bwd")
        if need_grad:
            gemm.linear_dgrad(dlogits[:n], w, out=dh[s:e])
            gemm.linear_wgrad(dlogits[:n], hc, out=dw, accumulate=True)
    return {"ce_sum": sums[0], "z_sum": sums[1], "correct": sums[2], "valid": sums[3], "dh": dh, "dw": dw}


# ---- sigmoid output gate ----------------------------------------------------------------------------
def _gate_view(buf, off, hstride, H, hd):
    T = buf.shape[0]
    return torch.as_strided(buf, (T, H, hd), (buf.stride(0), hstride, 1), buf.storage_offset() + off)


def sigmoid_gate_fwd(a, proj, gate_off, gate_hstride, H, hd):
    """a [T, H*hd] * sigmoid(gate), gate read in place from the projection output `proj`."""
    T = a.shape[0]
    if not (_cuda(a, proj) and a.dtype == torch.bfloat16):
        g = _gate_view(proj, gate_off, gate_hstride, H, hd).float()
        return (a.float().view(T, H, hd) * torch.sigmoid(g)).view(T, H * hd).to(a.dtype)
    out = torch.empty_like(a)
    rc = _lib.lib().adana_sigmoid_gate_fwd(a.data_ptr(), proj.data_ptr(), proj.stride(0), gate_off, gate_hstride,
                                           out.data_ptr(), T, H, hd, _lib.stream_ptr())
    _lib.check_rc(rc, "adana_sigmoid_gate_fwd")
    return out


def sigmoid_gate_bwd(dout, a, proj, dproj, gate_off, gate_hstride, H, hd):
    """Returns da; writes dgate into `dproj` (projection layout)."""
    T = a.shape[0]
    if not (_cuda(a, proj, dout, dproj) and a.dtype == torch.bfloat16):
        g = _gate_view(proj, gate_off, gate_hstride, H, hd).float()
        s = torch.sigmoid(g)
        d3 = dout.float().view(T, H, hd)
        _gate_view(dproj, gate_off, gate_hstride, H, hd).copy_((d3 * a.float().view(T, H, hd) * s * (1 - s)).to(dproj.dtype))
        return (d3 * s).view(T, H * hd).to(a.dtype)
    da = torch.empty_like(a)
    rc = _lib.lib().adana_sigmoid_gate_bwd(dout.data_ptr(), a.data_ptr(), proj.data_ptr(), proj.stride(0), gate_off,
                                           gate_hstride, da.data_ptr(), dproj.data_ptr(), T, H, hd, _lib.stream_ptr())
    _lib.check_rc(rc, "adana_sigmoid_gate_bwd")
    return da
