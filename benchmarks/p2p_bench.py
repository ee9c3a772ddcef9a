#!/usr/bin/env python
"""Times the peer-memory data-plane kernels (csrc/comm_p2p.cu) and reports achieved bytes/s.

    python benchmarks/p2p_bench.py [--world 4] [--mib 256] [--iters 20]                 # one GPU, fake peers
    torchrun --nproc-per-node N benchmarks/p2p_bench.py --real [--mib 256]              # N GPUs, NVLink peers

* reduce-scatter + sum of squares: every rank reads its slice of every rank's fp32 gradient buffer (world x shard
  x 4 B read, shard x 4 B written) — over NVLink for the (world-1)/world remote part.
* fused optimizer step + weight push (Dana-Star-MK4): reads p, g, m, v, tau, writes p, m, v, tau (36 B per
  element) and stores the bf16 result into every rank's weight buffer (2 B x world per element).
With fake peers every "rank" is an allocation on this one GPU, so all traffic is local HBM and the figure is
compared with the measured HBM copy bandwidth; with `--real` the time is the max over ranks (CUDA events) and
the remote bytes are compared with the NVLink per-direction bandwidth.
"""
import argparse
import json
import os
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from adana_b200.ops import _lib, optim  # noqa: E402
from adana_b200.parallel.p2p import P2PPlane  # noqa: E402


def timeit(fn, iters, sync=lambda: None):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=4)
    ap.add_argument("--mib", type=int, default=256, help="size of the fp32 gradient buffer per rank")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--real", action="store_true")
    a = ap.parse_args()
    peaks = {}
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        peaks = json.loads(pk.read_text())
    n = a.mib * (1 << 20) // 4
    kw = dict(kind=optim.KIND_DANA_STAR, lr=3e-4, alpha=8 / 108, step=100, kappa=0.85, clipsnr=2.0, eps=1e-8,
              gamma3=1.0, wd_factor=0.9999, grad_scale=1.0, betas=(0.9, 0.95))
    if a.real:
        import torch.distributed as dist

        dist.init_process_group("nccl")
        rank, world = dist.get_rank(), dist.get_world_size()
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        n -= n % (64 * world)
        plane = P2PPlane.create(n * 4 + n * 2 + (1 << 20), torch.device("cuda"))
        planes, mine = [plane], 0
    else:
        rank, world = 0, a.world
        n -= n % (64 * world)
        planes = P2PPlane.fake(n * 4 + n * 2 + (1 << 20), world, "cuda")
        mine = 0
    shard = n // world
    grads = [pl.alloc(n, torch.float32) for pl in planes]
    weights = [pl.alloc(n, torch.bfloat16) for pl in planes]
    for g in grads:
        g.normal_()
    pl = planes[mine]
    out = torch.empty(shard, device="cuda")
    ss = torch.zeros(1, device="cuda")
    sync = (lambda: pl.barrier()) if a.real else (lambda: None)
    t_rs = timeit(lambda: pl.reduce_scatter_sumsq(grads[mine], rank * shard, out, ss), a.iters, sync)
    p, m = torch.randn(shard, device="cuda"), torch.zeros(shard, device="cuda")
    v, tau = torch.full((shard,), 1e-4, device="cuda"), torch.full((shard,), 0.3, device="cuda")
    clip = torch.tensor([1.0, 0.0], device="cuda")
    hyper = optim.make_hyper(**kw)
    t_opt = timeit(lambda: pl.opt_step_push(p, out, m, v, tau, weights[mine], rank * shard, hyper, clip), a.iters, sync)
    if a.real:
        import torch.distributed as dist

        tt = torch.tensor([t_rs, t_opt], device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        t_rs, t_opt = tt.tolist()
    rs_bytes = shard * 4 * (world + 1)
    opt_bytes = shard * (36 + 2 * world)
    row = {"mode": "nvlink peers" if a.real else "fake peers on one GPU", "world": world, "shard_mib": shard * 4 / 2 ** 20,
           "reduce_scatter_ms": round(t_rs, 4), "reduce_scatter_gbs": round(rs_bytes / t_rs / 1e6, 1),
           "opt_step_push_ms": round(t_opt, 4), "opt_step_push_gbs": round(opt_bytes / t_opt / 1e6, 1)}
    if a.real:
        row["reduce_scatter_remote_gbs"] = round(shard * 4 * (world - 1) / t_rs / 1e6, 1)
        row["push_remote_gbs"] = round(shard * 2 * (world - 1) / t_opt / 1e6, 1)
        row["nvlink_measured_gbs_per_direction"] = 770
    elif peaks.get("hbm_gbs"):
        row["reduce_scatter_of_measured_hbm"] = round(rs_bytes / t_rs / 1e6 / peaks["hbm_gbs"], 3)
        row["opt_step_push_of_measured_hbm"] = round(opt_bytes / t_opt / 1e6 / peaks["hbm_gbs"], 3)
    if rank == 0:
        print(json.dumps(row), flush=True)
    torch.cuda.synchronize()
    _lib.check_status()


if __name__ == "__main__":
    main()
