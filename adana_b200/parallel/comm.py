"""Collective layer of the sharded engine.

`Comm` wraps a process group and offers exactly the collectives the engine needs on flat
buffers: reduce-scatter (sum) of a gradient unit into the rank's shard, all-gather of updated
parameter shards, all-reduce of small tensors, barrier.  Two data planes sit behind it:

  * "torch": `torch.distributed` — NCCL on GPUs (the measured baseline), Gloo on CPU ranks
    (tests; Gloo lacks reduce-scatter, which is emulated with all-reduce + slice);
  * "p2p": the hand-written peer-memory kernels of `adana_b200/parallel/p2p.py`
    (one-shot pull all-gather / reduce-scatter over NVLink with bounded flag waits).

World size 1 short-circuits everything (copies only).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


class Comm:
    def __init__(self, group=None, plane: str = "torch"):
        self.group = group
        if dist.is_available() and dist.is_initialized():
            self.world = dist.get_world_size(group)
            self.rank = dist.get_rank(group)
            self.backend = dist.get_backend(group)
        else:
            self.world, self.rank, self.backend = 1, 0, "none"
        self.plane = plane if self.world > 1 else "none"
        self._p2p = None

    # ---- optional peer-memory data plane -------------------------------------------------------
    def enable_p2p(self, p2p_engine) -> None:
        self._p2p = p2p_engine
        self.plane = "p2p"

    # ---- collectives ---------------------------------------------------------------------------
    def reduce_scatter_sum(self, full: torch.Tensor, shard_out: torch.Tensor, async_op: bool = False):
        """shard_out = sum over ranks of full[rank*len(shard): (rank+1)*len(shard)]."""
        if self.world == 1:
            shard_out.copy_(full)
            return None
        if self.plane == "p2p" and self._p2p is not None and self._p2p.owns(full):
            return self._p2p.reduce_scatter_sum(full, shard_out)
        if self.backend == "gloo":
            w = dist.all_reduce(full, op=dist.ReduceOp.SUM, group=self.group, async_op=False)
            n = shard_out.numel()
            shard_out.copy_(full[self.rank * n:(self.rank + 1) * n])
            return None
        return dist.reduce_scatter_tensor(shard_out, full, op=dist.ReduceOp.SUM, group=self.group,
                                          async_op=async_op)

    def all_gather(self, shard: torch.Tensor, full_out: torch.Tensor, async_op: bool = False):
        if self.world == 1:
            if full_out.data_ptr() != shard.data_ptr():
                full_out.copy_(shard)
            return None
        if self.plane == "p2p" and self._p2p is not None and self._p2p.owns(full_out):
            return self._p2p.all_gather(shard, full_out)
        try:
            return dist.all_gather_into_tensor(full_out, shard, group=self.group, async_op=async_op)
        except (RuntimeError, NotImplementedError):
            n = shard.numel()
            parts = [full_out[i * n:(i + 1) * n] for i in range(self.world)]
            dist.all_gather(parts, shard, group=self.group)
            return None

    def all_reduce_sum(self, t: torch.Tensor, async_op: bool = False):
        if self.world == 1:
            return None
        return dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group, async_op=async_op)

    def all_reduce_max(self, t: torch.Tensor):
        if self.world == 1:
            return None
        return dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)

    def broadcast(self, t: torch.Tensor, src: int = 0):
        if self.world == 1:
            return None
        if self.group is None:
            return dist.broadcast(t, src=src, group=self.group)
        return dist.broadcast(t, group=self.group, group_src=src)      # `src` counts inside this group

    def barrier(self):
        if self.world > 1:
            dist.barrier(group=self.group)


def wait(work) -> None:
    if work is not None:
        work.wait()
