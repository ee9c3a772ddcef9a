#!/usr/bin/env python
"""Row-parallel linear + reduce-scatter over peer memory in its three variants (parallel/tensor_parallel.py:
"pull" = GEMM into a local bf16 partial, then every rank adds the rows it owns out of all partials over NVLink;
"push" = csrc/gemm_tcgen05.cu EPI_BF16_PUSH, the epilogue stores partial rows into per-source slots at the owner;
"atomic" = EPI_F32_RS, the epilogue adds fp32 rows with vector atomics) against the library baseline (the plain GEMM into
an fp32 tensor, then NCCL reduce_scatter_tensor), on the tensor-parallel shapes of Enoki-36 (o-proj and MLP c_proj).

    torchrun --nproc-per-node N --master-addr 127.0.0.1 benchmarks/gemm_rs_bench.py [--iters 20]

Roofline: the slower of FLOPs / measured GEMM peak and the bytes of partial rows that leave this
GPU (M * N * 2 * (N_ranks - 1) / N_ranks, bf16) / 770 GB/s measured per direction; CUDA events, max over ranks.  Both
variants include zeroing the output and, for the fused one, the two plane barriers that bracket the launch.
"""
import argparse
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from adana_b200.ops import _lib, gemm  # noqa: E402
from adana_b200.parallel.p2p import P2PPlane  # noqa: E402
from adana_b200.parallel.tensor_parallel import RowParallelLinear  # noqa: E402

SHAPES = [(16384, 2304, 2304), (16384, 2304, 9216)]          # M, N, full K (split over the ranks)


def timeit(fn, iters, pre):
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
    a = ap.parse_args()
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    dist.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    for (M, N, K) in SHAPES:
        Kl = K // world
        x = (torch.randn(M, Kl, device="cuda") * 0.5).bfloat16()
        w = (torch.randn(N, Kl, device="cuda") * 0.5).bfloat16()
        plane = P2PPlane.create((M // world) * N * 4 + 2 * M * N * 2 + (1 << 16), torch.device("cuda"))
        op = RowParallelLinear(plane, M, N, mode="push")
        op_atomic = RowParallelLinear(plane, M, N, mode="atomic")
        op_pull = RowParallelLinear(plane, M, N, mode="pull")
        partial = torch.empty(M, N, device="cuda", dtype=torch.float32)
        shard = torch.empty(M // world, N, device="cuda", dtype=torch.float32)

        def baseline():
            gemm.linear_fwd_f32(x, w, out=partial)
            dist.reduce_scatter_tensor(shard, partial)

        t_fused = timeit(lambda: op(x, w), a.iters, plane.barrier)
        t_atomic = timeit(lambda: op_atomic(x, w), a.iters, plane.barrier)
        t_pull = timeit(lambda: op_pull(x, w), a.iters, plane.barrier)
        t_base = timeit(baseline, a.iters, plane.barrier)
        t_gemm = timeit(lambda: gemm.linear_fwd_f32(x, w, out=partial), a.iters, plane.barrier)
        tt = torch.tensor([t_fused, t_base, t_gemm, t_atomic, t_pull], device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        t_fused, t_base, t_gemm, t_atomic, t_pull = tt.tolist()
        flops = 2.0 * M * N * Kl
        out_bytes = M * N * 2 * (world - 1) / world       # bf16 partial rows that leave this GPU
        row = {"world": world, "M": M, "N": N, "K_local": Kl, "fused_push_ms": round(t_fused, 4),
               "fused_fp32_atomics_ms": round(t_atomic, 4), "gemm_then_own_pull_reduce_scatter_ms": round(t_pull, 4),
               "gemm_then_nccl_reduce_scatter_ms": round(t_base, 4), "gemm_alone_ms": round(t_gemm, 4),
               "nvlink_mb_out": round(out_bytes / 1e6, 1)}
        if peaks.get("bf16_tflops"):
            t_roof = max(flops / (peaks["bf16_tflops"] * 1e9), out_bytes / 770e6)
            row["roofline_ms"] = round(t_roof, 4)
            row["of_roofline"] = round(t_roof / min(t_fused, t_pull), 3)
        if rank == 0:
            print(json.dumps(row), flush=True)
        plane.barrier()
    torch.cuda.synchronize()
    _lib.check_status()


if __name__ == "__main__":
    main()
