#!/usr/bin/env python
"""Bandwidth-bound kernels of the training step against the measured HBM copy rate: LayerNorm / RMSNorm forward and
backward, per-head QK-norm + RoPE forward and backward, embedding forward and backward, the fused ADana-family
optimizer step, and the chunked linear + cross-entropy head (reported in FLOP/s as well: it is GEMM-bound at d = 2304).

    python benchmarks/membound_bench.py [--iters 20]

Shapes are the Enoki-36 micro-batch: 8 x 2048 tokens, d = 2304, 36 heads of 64, V = 50304.  Bytes are the
algorithmic ones (each tensor read or written once); inputs exceed the 126 MB L2 except where noted, and the timed
loop rotates over several input sets so that no call finds its data in L2.  Times are CUDA events after warm-up.
"""
import argparse
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from adana_b200.ops import _lib, misc, norm, optim, rope  # noqa: E402


def timeit(fns, iters):
    """fns: callables on different buffers, used round-robin."""
    for f in fns:
        f()
    for f in fns:
        f()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fns[i % len(fns)]()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=24)
    a = ap.parse_args()
    dev = torch.device("cuda")
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    hbm = peaks.get("hbm_gbs", 6650.0)
    tf = peaks.get("bf16_tflops", 1590.0)
    T, d, H, hd, V, S = 16384, 2304, 36, 64, 50304, 2048
    SETS = 4       # input sets rotated through: 4 x (>= 75 MB) > L2
    rows = []

    def report(name, ms, nbytes, flops=None, note=""):
        r = {"kernel": name, "ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1),
             "of_measured_hbm": round(nbytes / ms / 1e6 / hbm, 3)}
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 1)
            r["of_measured_gemm"] = round(flops / ms / 1e9 / tf, 3)
        if note:
            r["note"] = note
        rows.append(r)
        print(json.dumps(r), flush=True)

    for kind, kname in ((norm.LAYERNORM, "layernorm"), (norm.RMSNORM, "rmsnorm")):
        xs = [torch.randn(T, d, device=dev) for _ in range(SETS)]
        w = torch.rand(d, device=dev) + 0.5
        ms = timeit([lambda x=x: norm.norm_fwd(x, w, 1e-5, kind) for x in xs], a.iters)
        report(f"{kname} fwd (fp32 residual stream in, bf16 out)", ms, T * d * (4 + 2))
        stats = [norm.norm_fwd(x, w, 1e-5, kind) for x in xs]
        dys = [torch.randn(T, d, device=dev).bfloat16() for _ in range(SETS)]
        accs = [torch.randn(T, d, device=dev) for _ in range(SETS)]
        dw = torch.zeros(d, device=dev)
        fns = [lambda i=i: norm.norm_bwd(dys[i], xs[i], w, stats[i][1], stats[i][2], kind, dx_accum=accs[i], dw_out=dw,
                                         dw_accumulate=True) for i in range(SETS)]
        ms = timeit(fns, a.iters)
        # dy bf16 + x fp32 read, dx fp32 read-modify-write (the residual-stream gradient accumulates in place)
        report(f"{kname} bwd (+= into the fp32 stream gradient, weight-gradient partials + fold)", ms, T * d * (2 + 4 + 8))
        del xs, dys, accs, stats

    # per-head QK-norm + RoPE on the fused QKV projection output
    width = 3 * H * hd
    qkvs = [torch.randn(T, width, device=dev).bfloat16() for _ in range(SETS)]
    wq, wk = torch.rand(hd, device=dev) + 0.5, torch.rand(hd, device=dev) + 0.5
    freqs = rope.precompute_freqs_cis(hd, S).to(dev)
    args = (0, hd, H * hd, hd, wq, wk, freqs, S, H, H, hd, 1e-5, norm.LAYERNORM)
    ms = timeit([lambda q=q: rope.qknorm_rope_fwd(q, *args) for q in qkvs], a.iters)
    report("qk-layernorm + rope fwd (q, k of 36 heads x 64)", ms, 2 * T * H * hd * (2 + 2))
    dqs = [torch.randn(T, H, hd, device=dev).bfloat16() for _ in range(SETS)]
    dks = [torch.randn(T, H, hd, device=dev).bfloat16() for _ in range(SETS)]
    dqkvs = [torch.zeros(T, width, device=dev, dtype=torch.bfloat16) for _ in range(SETS)]
    ms = timeit([lambda i=i: rope.qknorm_rope_bwd(dqs[i], dks[i], qkvs[i], dqkvs[i], *args) for i in range(SETS)], a.iters)
    report("qk-layernorm + rope bwd", ms, 2 * T * H * hd * (2 + 2 + 2))
    del qkvs, dqs, dks, dqkvs

    # embedding
    table = torch.randn(V, d, device=dev)
    zipf = torch.distributions.Categorical(probs=1.0 / torch.arange(1, V + 1, dtype=torch.float64))
    idxs = [zipf.sample((T,)).to(dev) for _ in range(SETS)]
    ms = timeit([lambda i=i: misc.embedding_fwd(i, table) for i in idxs], a.iters)
    report("embedding fwd (fp32 table -> fp32 stream, Zipf tokens)", ms, T * d * (4 + 4))
    douts = [torch.randn(T, d, device=dev) for _ in range(SETS)]
    dtable = torch.zeros(V, d, device=dev)
    ms = timeit([lambda i=i: misc.embedding_bwd(idxs[i], douts[i], dtable) for i in range(SETS)], a.iters)
    report("embedding bwd (vector red.add into the fp32 table gradient)", ms, T * d * (4 + 8))
    del table, douts, dtable

    # optimizer: one flat range of 64 Mi parameters (fp32 p, g, m, v, tau read; p, m, v, tau written; bf16 copy written)
    n = 64 << 20
    p, gg, m = torch.randn(n, device=dev), torch.randn(n, device=dev) * 1e-2, torch.zeros(n, device=dev)
    v, tau = torch.rand(n, device=dev) * 1e-4, torch.rand(n, device=dev) * 0.5
    p16 = torch.empty(n, device=dev, dtype=torch.bfloat16)
    clip = torch.ones(1, device=dev)
    for kind, kname, nbytes in ((optim.KIND_DANA_STAR, "dana-star-mk4", n * (5 * 4 + 4 * 4 + 2)),
                                (optim.KIND_ADANA, "adana / dana-mk4", n * (4 * 4 + 3 * 4 + 2)),
                                (optim.KIND_ADAMW, "adamw", n * (4 * 4 + 3 * 4 + 2))):
        kw = dict(kind=kind, lr=3e-3, alpha=0.5, step=7, kappa=0.85, clipsnr=2.0, eps=1e-8, gamma3=1.0, wd_factor=0.999,
                  grad_scale=0.125, betas=(0.9, 0.95))
        ms = timeit([lambda: optim.fused_step(p, gg, m, v, tau if kind == optim.KIND_DANA_STAR else None, p16,
                                              clip_coef_t=clip, **kw)], a.iters)
        report(f"fused optimizer step, {kname} (64 Mi parameters, bf16 weight copy written)", ms, nbytes)
    del p, gg, m, v, tau, p16

    # LM head: chunked linear + cross-entropy + z-loss (logits never stored whole); forward, dh, dW
    h = (torch.randn(T, d, device=dev) * 0.5).bfloat16()
    w = (torch.randn(V, d, device=dev) * 0.02).bfloat16()
    tgt = torch.randint(0, V, (T,), device=dev)
    dwbuf = torch.zeros(V, d, device=dev)
    for chunk in (4096, 8192, 16384):
        ms = timeit([lambda: misc.linear_ce(h, w, tgt, z_coeff=1e-4, loss_scale=1.0 / T, dw_out=dwbuf, chunk_rows=chunk)],
                    max(4, a.iters // 4))
        report(f"linear + cross-entropy + z-loss, forward and both gradients (V = 50304), {chunk}-row chunks", ms,
               T * V * 2 * 5 + (T // chunk) * V * d * 8, flops=3 * 2.0 * T * V * d,
               note="bytes: bf16 logits written, read and rewritten as dlogits, read by two GEMMs; the fp32 weight gradient "
                    "read and written once per chunk")
    torch.cuda.synchronize()
    _lib.check_status()


if __name__ == "__main__":
    main()
