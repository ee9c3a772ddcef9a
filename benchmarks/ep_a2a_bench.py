#!/usr/bin/env python
"""Expert-parallel token exchange: the pull-style all-to-all over peer memory (parallel/p2p.py::P2PAllToAll,
csrc/comm_p2p.cu: p2p_all_to_all_pull_kernel) against NCCL (`all_to_all_single` of the counts, a host read, then
`all_to_all_single` of the rows), for T tokens x top-k routed uniformly over the experts.

    torchrun --nproc-per-node N --master-addr 127.0.0.1 benchmarks/ep_a2a_bench.py [--tokens 16384 --k 2 --d 2048]

Both variants include what they need to know the receive size (the peer-memory one reads it from the peers' tables).
Bytes = rows that leave this GPU x row size; link rate for the fraction: 770 GB/s measured per direction.  CUDA events,
max over ranks.
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
from adana_b200.ops import _lib  # noqa: E402
from adana_b200.parallel.p2p import P2PAllToAll, P2PPlane  # noqa: E402


def timeit(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--k", type=int, default=2)
    ap.add_argument("--d", type=int, default=2048)
    ap.add_argument("--experts_per_rank", type=int, default=4)
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    dist.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda")
    n_exp = world * a.experts_per_rank
    rows = a.tokens * a.k
    torch.manual_seed(rank)
    dest = torch.sort(torch.randint(0, n_exp, (rows,), device=dev)).values
    counts = torch.bincount(dest, minlength=n_exp)
    x = torch.randn(rows, a.d, device=dev).bfloat16()
    max_rows = 2 * rows
    plane = P2PPlane.create(P2PAllToAll.arena_bytes(max_rows, a.d, torch.bfloat16, world, a.experts_per_rank), dev)
    a2a = P2PAllToAll(plane, max_rows, a.d, torch.bfloat16, a.experts_per_rank)

    def ours():
        return a2a.exchange(x, counts)

    def nccl():
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts)
        in_splits = counts.view(world, -1).sum(1).tolist()
        out_splits = recv_counts.view(world, -1).sum(1).tolist()
        out = x.new_empty((sum(out_splits), a.d))
        dist.all_to_all_single(out, x, output_split_sizes=out_splits, input_split_sizes=in_splits)
        return out, recv_counts

    o1, c1 = ours()
    o2, c2 = nccl()
    same = bool(torch.equal(o1, o2) and torch.equal(c1.long(), c2.long()))
    t_ours, t_nccl = timeit(ours, a.iters), timeit(nccl, a.iters)
    tt = torch.tensor([t_ours, t_nccl], device=dev)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    t_ours, t_nccl = tt.tolist()
    remote_rows = rows - int(counts.view(world, -1)[rank].sum())
    nbytes = remote_rows * a.d * 2
    if rank == 0:
        print(json.dumps({"world": world, "rows": rows, "d": a.d, "same_result_as_nccl": same,
                          "p2p_pull_ms": round(t_ours, 4), "nccl_ms": round(t_nccl, 4),
                          "remote_mb": round(nbytes / 1e6, 1), "p2p_gbs": round(nbytes / t_ours / 1e6, 1),
                          "of_measured_770_gbs": round(nbytes / t_ours / 1e6 / 770, 3)}), flush=True)
    torch.cuda.synchronize()
    _lib.check_status()
    dist.barrier()


if __name__ == "__main__":
    main()
