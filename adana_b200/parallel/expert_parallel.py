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

On B200s of one node the two exchanges run over the peer-memory plane instead of NCCL (`P2PAllToAll`,
csrc/comm_p2p.cu: every rank publishes its sorted rows and its count table in symmetric memory and the receivers pull
their groups over NVLink), which also delivers the counts, so the separate count all-to-all disappears.  The ranks
agree on the path once, at the first forward; `ADANA_EP_COMM=nccl` keeps NCCL.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn as nn

from ..models.moe import _route


_EP_GROUPS = {}


def default_ep_group():
    """A process group of all ranks that only the expert exchange uses.  The exchange runs inside forward AND backward;
    on the default group its collectives would interleave with the gradient all-reduces that DistributedDataParallel
    issues from its own hooks during the same backward, and the two orders differ between ranks (a collective
    mismatch).  Created once, by every rank, the first time a layer is built."""
    if "world" not in _EP_GROUPS:
        _EP_GROUPS["world"] = dist.new_group(ranks=list(range(dist.get_world_size())))
    return _EP_GROUPS["world"]


def rank_local_parameters(model):
    """Names of the parameters that differ between ranks on purpose (each rank's own experts): data parallelism must
    neither broadcast nor all-reduce them."""
    return [n for n, p in model.named_parameters() if getattr(p, "_adana_rank_local", False)]


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


class _P2PExchange(torch.autograd.Function):
    """One `P2PAllToAll.exchange`; its backward is the reverse exchange with the received counts as the table."""

    @staticmethod
    def forward(ctx, x, seg_counts, a2a, expect_rows):
        out, recv_counts = a2a.exchange(x.contiguous(), seg_counts, expect_rows)
        ctx.a2a, ctx.recv_counts, ctx.n_in = a2a, recv_counts, x.shape[0]
        ctx.mark_non_differentiable(recv_counts)
        return out, recv_counts

    @staticmethod
    def backward(ctx, g, _):
        back, _ = ctx.a2a.exchange(g.contiguous(), ctx.recv_counts, ctx.n_in)
        return back, None, None, None


class ExpertParallelMoE(nn.Module):
    def __init__(self, config, mlp, group=None):
        super().__init__()
        if group is None and dist.is_initialized() and dist.get_world_size() > 1:
            group = default_ep_group()
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
        self._a2a = {}            # (dtype, width) -> P2PAllToAll, or None once the ranks settled on NCCL
        self._p2p_ok = None
        if self.world > 1:
            # This rank's experts exist nowhere else.  Through the exchange their gradients already sum the
            # contributions of every rank's loss; data parallelism averages the replicated parameters' gradients over the
            # ranks, so these are divided by the number of ranks to stay on the same scale.
            w = float(self.world)
            for p in self.experts.parameters():
                p._adana_rank_local = True
                p.register_hook(lambda g, w=w: g / w)

    def _p2p_exchange(self, x, rows_per_call: int):
        """The peer-memory exchange for rows like `x`, created on first use; None where NCCL is to be used.  Every
        rank must take the same path, so the outcome of the set-up is agreed with one all-reduce."""
        import os

        if self._p2p_ok is False or self.world <= 1:
            return None
        key = (x.dtype, x.shape[1])
        if key in self._a2a:
            return self._a2a[key]
        ok, a2a = 0, None
        try:
            from ..ops import _lib
            from .p2p import P2PAllToAll, P2PPlane

            usable = (x.is_cuda and _lib.available() and self.world <= 8 and dist.get_backend(self.group) == "nccl"
                      and os.environ.get("ADANA_EP_COMM", "p2p") != "nccl" and (x.shape[1] * x.element_size()) % 16 == 0
                      and _lib.has("adana_p2p_all_to_all_pull"))
            if usable:
                # worst case every token of every rank comes here; cap the buffer at 2 GiB
                per_row = x.shape[1] * x.element_size()
                mult = max(1, min(self.world, (2 << 30) // max(1, rows_per_call * per_row)))
                max_rows = rows_per_call * mult
                # (the symmetric-memory rendezvous happens once, here, outside any backward: the exchange's own group
                # has the same ranks as the default one, which is the one this set-up has always been run with)
                plane_group = None if self.group is _EP_GROUPS.get("world") else self.group
                plane = P2PPlane.create(P2PAllToAll.arena_bytes(max_rows, x.shape[1], x.dtype, self.world, self.per_rank),
                                        x.device, group=plane_group)
                a2a = P2PAllToAll(plane, max_rows, x.shape[1], x.dtype, self.per_rank)
                ok = 1
        except Exception:      # no symmetric memory here: all ranks fall back together below
            ok, a2a = 0, None
        flag = torch.tensor([ok], device=x.device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 0:
            self._p2p_ok, a2a = False, None
        else:
            self._p2p_ok = True
        self._a2a[key] = a2a
        return a2a

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
        a2a = self._p2p_exchange(x, T * k) if self.world > 1 else None
        if a2a is not None:
            return self._forward_p2p(inputs, x, logits, weights, selected, order, tok, send_counts, a2a)
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
        y = self._run_experts(recv, recv_counts)
        back = _AllToAll.apply(y, in_splits, out_splits, self.group) if self.world > 1 else y
        return self._combine(inputs, x, logits, weights, selected, order, tok, back)

    def _run_experts(self, recv, recv_counts):
        """Rows arrive grouped by source rank, then by local expert: run each expert on its rows."""
        x = recv
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
        return y

    def _forward_p2p(self, inputs, x, logits, weights, selected, order, tok, send_counts, a2a):
        recv, recv_counts = _P2PExchange.apply(x[tok], send_counts, a2a, None)
        y = self._run_experts(recv, recv_counts)
        back, _ = _P2PExchange.apply(y, recv_counts, a2a, tok.numel())
        return self._combine(inputs, x, logits, weights, selected, order, tok, back)

    def _combine(self, inputs, x, logits, weights, selected, order, tok, back):
        w = weights.reshape(-1)[order].to(x.dtype)
        out = torch.zeros_like(x).index_add(0, tok, back * w[:, None])
        for e in self.shared:
            out = out + e(x)[0]
        return out.view_as(inputs), {"router_logits": logits, "selected_experts": selected}
