#!/usr/bin/env python
"""Causal attention sweep: forward (and backward / forward-mode tangent when built) of the
hand-written tcgen05 kernels against PyTorch SDPA (library comparator), bf16, seeded N(0,1) inputs.

    python benchmarks/attention_bench.py [--B 8] [--heads 12 16 36] [--hd 64 128] [--S 1024 2048 4096 8192]
                                         [--what fwd bwd jvp] [--iters 10]

TFLOP/s counts the causal half: forward 4*B*H*S^2*hd/2, backward 2.5x that, JVP 3x (six GEMM chains per tile).
"""
import argparse
import json
import math
import sys
from pathlib import Path

import torch
import torch.nn.functional as F

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from adana_b200.ops import _lib, attention_native  # noqa: E402


def timeit(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--B", type=int, default=8)
    ap.add_argument("--heads", type=int, nargs="+", default=[12, 16, 36])
    ap.add_argument("--hd", type=int, nargs="+", default=[64, 128])
    ap.add_argument("--S", type=int, nargs="+", default=[1024, 2048, 4096, 8192])
    ap.add_argument("--what", nargs="+", default=["fwd", "bwd"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--jvp_comparator", action="store_true", help="also time torch.func.jvp over math attention (S <= 2048)")
    a = ap.parse_args()
    torch.manual_seed(0)
    for hd in a.hd:
        for H in a.heads:
            for S in a.S:
                B = a.B
                T = B * S
                qkv = torch.randn(T, 3 * H * hd, device="cuda").bfloat16()
                q = torch.randn(T, H, hd, device="cuda").bfloat16()
                k = torch.randn(T, H, hd, device="cuda").bfloat16()
                v_off = 2 * H * hd
                scale = 1.0 / math.sqrt(hd)
                flops_fwd = 4.0 * B * H * S * S * hd / 2
                q4 = q.view(B, S, H, hd).transpose(1, 2)
                k4 = k.view(B, S, H, hd).transpose(1, 2)
                v4 = torch.as_strided(qkv, (B, H, S, hd), (S * qkv.stride(0), hd, qkv.stride(0), 1), v_off)
                row = {"B": B, "H": H, "hd": hd, "S": S}
                if "fwd" in a.what:
                    t = timeit(lambda: attention_native.fwd(q, k, qkv, v_off, hd, B, S, scale), a.iters)
                    tl = timeit(lambda: F.scaled_dot_product_attention(q4, k4, v4, is_causal=True, scale=scale), a.iters)
                    row.update(fwd_ms=round(t, 4), fwd_tflops=round(flops_fwd / t / 1e9, 1),
                               sdpa_fwd_ms=round(tl, 4), sdpa_fwd_tflops=round(flops_fwd / tl / 1e9, 1))
                if "bwd" in a.what and attention_native.bwd_available():
                    out, lse2 = attention_native.fwd(q, k, qkv, v_off, hd, B, S, scale)
                    do = torch.randn_like(out)
                    dqkv = torch.empty_like(qkv)
                    t = timeit(lambda: attention_native.bwd(do, q, k, qkv, v_off, hd, B, S, scale, lse2, out, dqkv), a.iters)
                    qd, kd, vd = (x.detach().requires_grad_(True) for x in (q4, k4, v4))
                    o = F.scaled_dot_product_attention(qd, kd, vd, is_causal=True, scale=scale)
                    g = torch.randn_like(o)
                    tl = timeit(lambda: torch.autograd.grad(o, (qd, kd, vd), g, retain_graph=True), a.iters)
                    row.update(bwd_ms=round(t, 4), bwd_tflops=round(2.5 * flops_fwd / t / 1e9, 1),
                               sdpa_bwd_ms=round(tl, 4), sdpa_bwd_tflops=round(2.5 * flops_fwd / tl / 1e9, 1))
                if "jvp" in a.what and attention_native.jvp_available():
                    v = torch.randn(T, H, hd, device="cuda").bfloat16()
                    tq, tk, tv = (torch.randn(T, H, hd, device="cuda").bfloat16() for _ in range(3))
                    t = timeit(lambda: attention_native.jvp(q, k, v, tq, tk, tv, B, S, scale), a.iters)
                    row.update(jvp_ms=round(t, 4), jvp_tflops=round(3.0 * flops_fwd / t / 1e9, 1))
                    if a.jvp_comparator and S <= 2048:
                        # comparator: torch.func.jvp over the math attention (fp32 scores are materialised)
                        vv4 = v.view(B, S, H, hd).transpose(1, 2)
                        tq4, tk4, tv4 = (x.view(B, S, H, hd).transpose(1, 2) for x in (tq, tk, tv))

                        def math_attn(q_, k_, v_):
                            s_ = (q_ @ k_.transpose(-1, -2)) * scale
                            s_ = s_.masked_fill(~torch.ones(S, S, dtype=torch.bool, device="cuda").tril(), float("-inf"))
                            return torch.softmax(s_, -1) @ v_

                        tl = timeit(lambda: torch.func.jvp(math_attn, (q4, k4, vv4), (tq4, tk4, tv4)), max(2, a.iters // 3))
                        row.update(torch_jvp_ms=round(tl, 4), torch_jvp_tflops=round(3.0 * flops_fwd / tl / 1e9, 1))
                print(json.dumps(row), flush=True)
    torch.cuda.synchronize()
    _lib.check_status()


if __name__ == "__main__":
    main()
