#!/usr/bin/env python
"""All-gather fused into the GEMM (csrc/gemm_tcgen05.cu: gemm_bf16_gather_staged_kernel, which brings every remote
slice over the link once while the tiles of the local slice run; `direct_fetch_ms` is gemm_bf16_gather_kernel, which
re-fetches remote tiles per row tile) against the unfused baseline (NCCL all-gather of the weight shards, then the
plain GEMM), on the Enoki-36 projection shapes.

    torchrun --nproc-per-node N --master-addr 127.0.0.1 benchmarks/gather_gemm_bench.py [--iters 20]
    python benchmarks/gather_gemm_bench.py --fake 8          # one GPU: shards are separate local allocations

Roofline of the fused kernel: the slower of FLOPs / measured GEMM peak and remote weight bytes / NVLink rate
(770 GB/s measured per direction); times are CUDA events, max over ranks.
"""
import argparse
import json
import os
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from adana_b200.ops import _lib, gemm  # noqa: E402

# M, weight rows, weight columns, dgrad?  forward: y [M, rows] = x [M, cols] W^T; dgrad: dx [M, cols] = dy [M, rows] W
SHAPES = [(16384, 6912, 2304, False), (16384, 9216, 2304, False), (16384, 2304, 9216, False),
          (16384, 2304, 2304, False), (16384, 9216, 2304, True), (16384, 2304, 9216, True)]


def timeit(fn, iters, pre=lambda: None):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    pre()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--fake", type=int, default=0, help="emulate this many ranks with local allocations on one GPU")
    a = ap.parse_args()
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    real = a.fake == 0
    if real:
        import torch.distributed as dist

        from adana_b200.parallel.p2p import P2PPlane

        dist.init_process_group("nccl")
        rank, world = dist.get_rank(), dist.get_world_size()
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    else:
        rank, world = 0, a.fake
    for (M, N, K, dgrad) in SHAPES:
        starts = gemm.tile_aligned_row_starts(N, world)      # slices cut on whole 128-row tiles (uneven)
        rps = max(b - a for a, b in zip(starts, starts[1:]))  # allocation size per rank
        x = (torch.randn(M, N if dgrad else K, device="cuda") * 0.5).bfloat16()
        y = torch.empty(M, K if dgrad else N, device="cuda", dtype=torch.bfloat16)
        full = torch.empty(N, K, device="cuda", dtype=torch.bfloat16)

        def plain():
            return gemm.linear_dgrad(x, full, out=y) if dgrad else gemm.linear_fwd(x, full, out=y)

        if real:
            plane = P2PPlane.create(rps * K * 2 + (1 << 16), torch.device("cuda"))
            mine = plane.alloc(rps * K, torch.bfloat16).view(rps, K)
            mine.normal_(0, 0.5)
            torch.cuda.synchronize()
            plane.barrier()
            ptrs = plane.peer_ptrs(mine)
            sync = plane.barrier
            padded = torch.empty(world * rps, K, device="cuda", dtype=torch.bfloat16)

            def baseline():
                dist.all_gather_into_tensor(padded.view(-1), mine.view(-1))
                for r in range(world):      # compact the (slightly uneven) slices into the weight matrix
                    full[starts[r]:starts[r + 1]].copy_(padded[r * rps:r * rps + starts[r + 1] - starts[r]])
                plain()
        else:
            shards = [(torch.randn(b - a_, K, device="cuda") * 0.5).bfloat16() for a_, b in zip(starts, starts[1:])]
            ptrs, mine, sync = shards, shards[0], (lambda: None)

            def baseline():
                torch.cat(shards, out=full)
                plain()

        def fused(staged):
            if dgrad:
                return gemm.linear_dgrad_gathered(x, ptrs, None, K, out=y, row_starts=starts, me=rank, staged=staged)
            return gemm.linear_fwd_gathered(x, ptrs, None, out=y, row_starts=starts, me=rank, staged=staged)

        t_fused = timeit(lambda: fused(True), a.iters, sync)
        t_direct = timeit(lambda: fused(False), a.iters, sync)
        t_base = timeit(baseline, a.iters, sync)
        t_plain = timeit(plain, a.iters, sync)
        if real:
            tt = torch.tensor([t_fused, t_base, t_plain, t_direct], device="cuda")
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            t_fused, t_base, t_plain, t_direct = tt.tolist()
            plane.barrier()
        flops = 2.0 * M * N * K
        remote = (N - (starts[rank + 1] - starts[rank])) * K * 2
        row = {"mode": "nvlink peers" if real else "local shards", "world": world, "M": M,
               "weight": [N, K], "op": "dgrad" if dgrad else "forward",
               "fused_ms": round(t_fused, 4), "fused_tflops": round(flops / t_fused / 1e9, 1),
               "direct_fetch_ms": round(t_direct, 4),
               "allgather_then_gemm_ms": round(t_base, 4), "resident_gemm_ms": round(t_plain, 4),
               "remote_weight_mb": round(remote / 1e6, 1)}
        if peaks.get("bf16_tflops"):
            t_roof = max(flops / (peaks["bf16_tflops"] * 1e9), remote / 770e6 if real else 0.0)
            row["roofline_ms"] = round(t_roof, 4)
            row["of_roofline"] = round(t_roof / t_fused, 3)
        if rank == 0:
            print(json.dumps(row), flush=True)
    torch.cuda.synchronize()
    _lib.check_status()


if __name__ == "__main__":
    main()
