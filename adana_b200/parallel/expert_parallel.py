"""Expert-parallel MoE: the routed experts are split over the ranks (E/N each), the router is
replicated, tokens travel to the rank that owns their expert and come back weighted.

Dispatch is drop-free and exact: (token, choice) pairs are sorted by destination expert, the ranks
exchange per-expert counts, and ONE variable-size all-to-all carries the activations each way.  Both
exchanges are autograd functions (the backward of an all-to-all is the all-to-all with the split sizes
swapped), so expert and router gradients flow across ranks — the reference's version
(src/models/moe_expert_parallel.py:31-344) used padded capacity buffers, five fixed-size all-to-alls
per layer and plain c10d calls that cut the graph.  `capacity_factor` is accepted for compatibility;
when set > 0 tokens beyond `ceil(cf * T * k / E)` per expert are dropped like upstream.
On Gloo (CPU tests) the exchange falls back to all-gather + select.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn as nn

from ..models.moe import _route


def _all_to_all(x, out_splits, in_splits, group):
    out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
    if dist.get_backend(group) == "gloo":
        # emulate with all_gather: every rank publishes its send buffer and split table
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        sizes = [torch.zeros(1, dtype=torch.long) for _ in range(world)]
        dist.all_gather(sizes, torch.tensor([x.shape[0]]), group=group)
        maxn = max(int(s) for s in sizes)
        pad = x.new_zeros((maxn,) + tuple(x.shape[1:]))
        pad[:x.shape[0]] = x
        bufs = [torch.empty_like(pad) for _ in range(world)]
        dist.all_gather(bufs, pad, group=group)
        tables = [torch.zeros(world, dtype=torch.long) for _ in range(world)]
        dist.all_gather(tables, torch.tensor(in_splits, dtype=torch.long), group=group)
        pos = 0
        for src in range(world):
            start = int(tables[src][:rank].sum())
            n = int(tables[src][rank])
            out[pos:pos + n] = bufs[src][start:start + n]
            pos += n
        return out
    dist.all_to_all_single(out, x.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
    return out


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.out_splits, ctx.in_splits, ctx.group = out_splits, in_splits, group
        return _all_to_all(x, out_splits, in_splits, group)

    @staticmethod
    def backward(ctx, g):
        return _all_to_all(g.contiguous(), ctx.in_splits, ctx.out_splits, ctx.group), None, None, None


class ExpertParallelMoE(nn.Module):
    def __init__(self, config, mlp, group=None):
        super().__init__()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        n_routed = config.moe_num_experts - config.moe_num_shared_experts
        assert n_routed % self.world == 0, f"{n_routed} routed experts do not split over {self.world} ranks"
        self.n_routed, self.per_rank = n_routed, n_routed // self.world
        self.n_shared_experts = config.moe_num_shared_experts
        self.shared = nn.ModuleList([mlp(config=config) for _ in range(self.n_shared_experts)])
        self.experts = nn.ModuleList([mlp(config=config) for _ in range(self.per_rank)])   # this rank's experts
        self.router = nn.Linear(config.n_embd, n_routed, bias=False)
        self.top_k = config.moe_num_experts_per_tok
        self.softmax_order = config.moe_softmax_order
        self.capacity_factor = float(getattr(config, "moe_expert_capacity_factor", 0.0) or 0.0)

    def forward(self, inputs):
        x = inputs.view(-1, inputs.shape[-1])
        T, k = x.shape[0], self.top_k
        logits = self.router(x)
        weights, selected = _route(logits, k, self.softmax_order)
        flat_e = selected.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        if self.capacity_factor > 0:      # optional token dropping, per expert, in arrival order
            cap = math.ceil(self.capacity_factor * T * k / self.n_routed)
            sorted_e = flat_e[order]
            first = torch.searchsorted(sorted_e, torch.arange(self.n_routed, device=x.device))
            keep = (torch.arange(order.numel(), device=x.device) - first[sorted_e]) < cap
            order = order[keep]
        tok = order // k
        sorted_e = flat_e[order]
        send_counts = torch.bincount(sorted_e, minlength=self.n_routed)
        if self.world > 1:
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts, group=self.group) if dist.get_backend(self.group) != "gloo" \
                else recv_counts.copy_(_all_to_all(send_counts, [self.per_rank] * self.world,
                                                   [self.per_rank] * self.world, self.group))
        else:
            recv_counts = send_counts
        in_splits = send_counts.view(self.world, self.per_rank).sum(1).tolist()
        out_splits = recv_counts.view(self.world, self.per_rank).sum(1).tolist()
        xs = x[tok]
        recv = _AllToAll.apply(xs, out_splits, in_splits, self.group) if self.world > 1 else xs
        # rows arrive grouped by source rank, then by local expert: run each expert on its rows
        per_src = recv_counts.view(self.world, self.per_rank).tolist()
        y = torch.empty_like(recv)
        pos = 0
        segments = [[] for _ in range(self.per_rank)]
        for src in range(self.world):
            for e in range(self.per_rank):
                n = per_src[src][e]
                if n:
                    segments[e].append((pos, n))
                pos += n
        for e, segs in enumerate(segments):
            if not segs:
                continue
            idx = torch.cat([torch.arange(s, s + n, device=x.device) for s, n in segs])
            out_e, _ = self.experts[e](recv[idx])
            y = y.index_copy(0, idx, out_e.to(y.dtype))
        back = _AllToAll.apply(y, in_splits, out_splits, self.group) if self.world > 1 else y
        w = weights.reshape(-1)[order].to(x.dtype)
        out = torch.zeros_like(x).index_add(0, tok, back * w[:, None])
        for e in self.shared:
            out = out + e(x)[0]
        return out.view_as(inputs), {"router_logits": logits, "selected_experts": selected}
