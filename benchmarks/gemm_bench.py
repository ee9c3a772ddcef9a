#!/usr/bin/env python
"""Times the tcgen05 GEMM (forward / dgrad / wgrad operand layouts) against torch.matmul (cuBLAS)
on the layer shapes of the flagship model and reports TFLOP/s and the fraction of the measured
cuBLAS peak (MEASURED_PEAKS.json when present).

    python benchmarks/gemm_bench.py [--shapes enoki36|square] [--iters 20] [--variant fwd|dgrad|wgrad|all] [--mode 0|1|2]

CUDA events on the launching stream, 3 warm-up calls, operands far larger than L2.
"""
import argparse
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from adana_b200.ops import _lib, gemm  # noqa: E402

SHAPES = {
    "enoki36": [(16384, 6912, 2304), (16384, 2304, 2304), (16384, 9216, 2304), (16384, 2304, 9216)],
    "square": [(8192, 8192, 8192), (4096, 4096, 4096)],
    "small": [(2048, 2304, 2304)],
}


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
    ap.add_argument("--shapes", default="enoki36", choices=sorted(SHAPES))
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--variant", default="all", choices=["fwd", "dgrad", "wgrad", "all"])
    ap.add_argument("--no_cublas", action="store_true")
    ap.add_argument("--mode", type=int, default=0, help="0 per shape, 1 one CTA per tile, 2 CTA pair per tile")
    a = ap.parse_args()
    gemm.set_mode(a.mode)
    peak = None
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        peak = json.loads(pk.read_text()).get("bf16_tflops")
    rows = []
    for (M, N, K) in SHAPES[a.shapes]:
        x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
        w = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
        dy = (torch.randn(M, N, device="cuda") * 0.5).bfloat16()
        y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        dx = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
        dw = torch.empty(N, K, device="cuda", dtype=torch.float32)
        variants = {
            "fwd": (lambda: gemm.linear_fwd(x, w, out=y), lambda: torch.matmul(x, w.t(), out=y)),
            "dgrad": (lambda: gemm.linear_dgrad(dy, w, out=dx), lambda: torch.matmul(dy, w, out=dx)),
            "wgrad": (lambda: gemm.linear_wgrad(dy, x, out=dw), lambda: torch.matmul(dy.t(), x)),
        }
        for name, (mine, lib) in variants.items():
            if a.variant not in ("all", name):
                continue
            t = timeit(mine, a.iters)
            tf = 2 * M * N * K / t / 1e9
            row = {"variant": name, "mode": a.mode, "M": M, "N": N, "K": K, "ms": round(t, 4), "tflops": round(tf, 1)}
            if not a.no_cublas:
                tl = timeit(lib, a.iters)
                row["cublas_tflops"] = round(2 * M * N * K / tl / 1e9, 1)
                row["vs_cublas"] = round(tl / t, 3)
            if peak:
                row["of_measured_peak"] = round(tf / peak, 3)
            rows.append(row)
            print(json.dumps(row), flush=True)
    torch.cuda.synchronize()
    _lib.check_status()


if __name__ == "__main__":
    main()
