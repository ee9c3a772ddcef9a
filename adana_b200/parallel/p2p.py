"""Peer-memory data plane: symmetric arena + the hand-written collectives of csrc/comm_p2p.cu.

Every rank allocates one arena through `torch.distributed._symmetric_memory`, the ranks exchange
handles once (`rendezvous`) and from then on every rank holds a device pointer to every other
rank's arena.  The engine places its gradient buffers, its resident bf16 weight buffers and the
fp32 norm-weight mirrors inside the arena, so "the same tensor on rank r" is `peer_base[r] + offset`
and the kernels read / write peers directly over NVLink:

    barrier()                       flag barrier with a bounded wait (status word on time-out)
    reduce_scatter_sumsq(...)       pull-reduce my shard from all ranks + squared-norm partial
    signal_unit / reduce_scatter_unit / all_reduce_unit
                                    per-unit "ready" flags instead of a barrier, bf16 or fp32 wire format
    global_clip_coef(...)           publish partials to all peers, barrier, sum locally
    opt_step_push(...)              fused optimizer step storing bf16 results into every rank's weights
    push_f32(...)                   exact fp32 copy of my slice of the norm weights to every rank

A fake-peer mode (`P2PPlane.fake(...)`: all "ranks" are allocations on one GPU) runs the same
kernels on a single device for tests; only kernels that do not wait on another rank are run there.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib

FLAG_BYTES = 32768      # uint32 flag slots at the start of the arena: [0, 64) barriers, then 8 per gradient unit
UNIT_FLAG_BASE = 64
SLOT_BYTES = 4096       # float slots for published scalars
ALIGN = 256


def _u64_array(vals):
    return (ctypes.c_ulonglong * len(vals))(*[int(v) for v in vals])


class P2PPlane:
    def __init__(self, rank: int, world: int, device, arena: torch.Tensor, peer_bases: List[int], timeout_s=20.0):
        self.rank, self.world, self.device = rank, world, torch.device(device)
        self.arena = arena
        self.peer_bases = peer_bases
        self.base = arena.data_ptr()
        self.cursor = FLAG_BYTES + SLOT_BYTES
        self.seq = 0
        self.timeout_ns = int(timeout_s * 1e9)
        self.stream = torch.cuda.Stream(device=self.device)
        self._flag_ptrs = _u64_array(peer_bases)
        self._slot_ptrs = _u64_array([b + FLAG_BYTES for b in peer_bases])
        self.slots = arena[FLAG_BYTES:FLAG_BYTES + SLOT_BYTES].view(torch.float32)
        self.handle = None

    # ---- construction ---------------------------------------------------------------------------------
    @classmethod
    def create(cls, nbytes: int, device, group=None, timeout_s=20.0) -> "P2PPlane":
        import torch.distributed._symmetric_memory as symm

        group = group or dist.group.WORLD
        total = nbytes + FLAG_BYTES + SLOT_BYTES + ALIGN
        arena = symm.empty(total, dtype=torch.uint8, device=device)
        arena.zero_()
        handle = symm.rendezvous(arena, group)
        plane = cls(dist.get_rank(group), dist.get_world_size(group), device, arena,
                    [int(p) for p in handle.buffer_ptrs], timeout_s)
        plane.handle = handle
        torch.cuda.synchronize(device)
        dist.barrier(group)
        return plane

    @classmethod
    def fake(cls, nbytes: int, world: int, device) -> List["P2PPlane"]:
        """`world` planes on ONE device whose "peers" are each other's arenas (single-GPU tests)."""
        total = nbytes + FLAG_BYTES + SLOT_BYTES + ALIGN
        arenas = [torch.zeros(total, dtype=torch.uint8, device=device) for _ in range(world)]
        bases = [a.data_ptr() for a in arenas]
        return [cls(r, world, device, arenas[r], bases) for r in range(world)]

    def alloc(self, numel: int, dtype) -> torch.Tensor:
        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        start = (self.cursor + ALIGN - 1) // ALIGN * ALIGN
        if start + nbytes > self.arena.numel():
            raise MemoryError("symmetric arena exhausted")
        self.cursor = start + nbytes
        return self.arena[start:start + nbytes].view(dtype)

    def owns(self, t: torch.Tensor) -> bool:
        return self.base <= t.data_ptr() < self.base + self.arena.numel()

    def peer_ptrs(self, t: torch.Tensor):
        off = t.data_ptr() - self.base
        return _u64_array([b + off for b in self.peer_bases])

    # ---- collectives (all enqueue on the current stream) -----------------------------------------------------
    def barrier(self):
        self.seq += 1
        rc = _lib.lib().adana_p2p_barrier(self._flag_ptrs, self.rank, self.world, 0, self.seq & 0xFFFFFFFF,
                                          self.timeout_ns, _lib.status_buffer(self.device).data_ptr(),
                                          _lib.stream_ptr())
        _lib.check_rc(rc, "adana_p2p_barrier")

    def reduce_scatter_sumsq(self, full: torch.Tensor, shard_off: int, shard_out: torch.Tensor, sumsq: Optional[torch.Tensor]):
        rc = _lib.lib().adana_p2p_reduce_scatter(self.peer_ptrs(full), self.world, shard_off, shard_out.numel(),
                                                 shard_out.data_ptr(), _lib.ptr(sumsq), _lib.stream_ptr())
        _lib.check_rc(rc, "adana_p2p_reduce_scatter")

    # ---- flag-ordered gradient collectives -----------------------------------------------------------------
    def unit_flag_slot(self, unit_index: int) -> int:
        slot = UNIT_FLAG_BASE + 8 * unit_index
        if (slot + 8) * 4 > FLAG_BYTES:
            raise ValueError(f"no flag slots left for gradient unit {unit_index}")
        return slot

    def signal_unit(self, unit_index: int, seq: int):
        """Tell every rank that this rank's copy of the unit is complete (everything enqueued on the current
        stream before this call)."""
        rc = _lib.lib().adana_p2p_signal(self._flag_ptrs, self.rank, self.world, self.unit_flag_slot(unit_index),
                                         seq & 0xFFFFFFFF, _lib.stream_ptr())
        _lib.check_rc(rc, "adana_p2p_signal")

    def _my_unit_flags(self, unit_index: int, wait: bool) -> int:
        return self.base + 4 * self.unit_flag_slot(unit_index) if wait else 0

    def reduce_scatter_unit(self, src_full: torch.Tensor, shard_off: int, shard_out: torch.Tensor,
                            sumsq: Optional[torch.Tensor], unit_index: int, seq: int, wait: bool = True):
        """shard_out (fp32) = sum over ranks of their `src_full` (fp32 or bf16, at the same arena offset) over my shard,
        once every rank has signalled the unit with sequence number `seq`; squared norm of the result added to `sumsq`."""
        rc = _lib.lib().adana_p2p_reduce_scatter_flag(
            self.peer_ptrs(src_full), int(src_full.dtype == torch.bfloat16), self._my_unit_flags(unit_index, wait),
            seq & 0xFFFFFFFF, self.world, shard_off, shard_out.numel(), shard_out.data_ptr(), _lib.ptr(sumsq),
            self.timeout_ns, _lib.status_buffer(self.device).data_ptr(), _lib.stream_ptr())
        _lib.check_rc(rc, "adana_p2p_reduce_scatter_flag")

    def all_reduce_unit(self, src_full: torch.Tensor, dst_full: torch.Tensor, slice_off: int, n: int, unit_index: int,
                        seq: int, wait: bool = True, sumsq: Optional[torch.Tensor] = None):
        """Slice [slice_off, slice_off + n) of every rank's `dst_full` (fp32) = sum over ranks of `src_full`; the
        squared norm of that slice of the result is added to `sumsq`."""
        rc = _lib.lib().adana_p2p_all_reduce_flag(
            self.peer_ptrs(src_full), int(src_full.dtype == torch.bfloat16), self.peer_ptrs(dst_full),
            self._my_unit_flags(unit_index, wait), seq & 0xFFFFFFFF, self.world, slice_off, n, _lib.ptr(sumsq), self.timeout_ns,
            _lib.status_buffer(self.device).data_ptr(), _lib.stream_ptr())
        _lib.check_rc(rc, "adana_p2p_all_reduce_flag")

    def global_clip_coef(self, local_sumsq: torch.Tensor, norm_scale: float, max_norm: float, out: torch.Tensor):
        """All ranks' squared-norm partials -> clip coefficient on the device (out[0]) and the norm (out[1])."""
        lib = _lib.lib()
        rc = lib.adana_p2p_publish_f32(self._slot_ptrs, self.rank, self.world, local_sumsq.data_ptr(), _lib.stream_ptr())
        _lib.check_rc(rc, "adana_p2p_publish_f32")
        self.barrier()
        rc = lib.adana_clip_coef_multi(self.slots.data_ptr(), self.world, float(norm_scale), float(max_norm),
                                       out.data_ptr(), _lib.stream_ptr())
        _lib.check_rc(rc, "adana_clip_coef_multi")

    def opt_step_push(self, p, g, m, v, tau, weights_full: torch.Tensor, push_off: int, hyper, clip_coef_t):
        rc = _lib.lib().adana_p2p_opt_step_push(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), _lib.ptr(tau),
                                                self.peer_ptrs(weights_full), self.world, push_off, p.numel(),
                                                ctypes.byref(hyper), _lib.ptr(clip_coef_t), _lib.stream_ptr())
        _lib.check_rc(rc, "adana_p2p_opt_step_push")

    def opt_step_push_to(self, p, g, m, v, tau, dst_ptrs, push_off: int, hyper, clip_coef_t):
        """Fused optimizer step whose bf16 results are stored at `push_off` into the buffers whose device addresses
        are given in `dst_ptrs` (own or peer memory) instead of into every rank's copy."""
        arr = _u64_array([int(x) for x in dst_ptrs])
        rc = _lib.lib().adana_p2p_opt_step_push(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), _lib.ptr(tau),
                                                arr, len(dst_ptrs), push_off, p.numel(), ctypes.byref(hyper),
                                                _lib.ptr(clip_coef_t), _lib.stream_ptr())
        _lib.check_rc(rc, "adana_p2p_opt_step_push")

    def push_f32(self, src: torch.Tensor, dst_full: torch.Tensor, dst_off: int):
        rc = _lib.lib().adana_p2p_push_f32(src.data_ptr(), self.peer_ptrs(dst_full), self.world, dst_off, src.numel(),
                                           _lib.stream_ptr())
        _lib.check_rc(rc, "adana_p2p_push_f32")


class P2PAllToAll:
    """Variable-size all-to-all of rows over the peer-memory plane, pull style (csrc/comm_p2p.cu:
    p2p_all_to_all_pull_kernel): the dispatch and combine exchanges of expert parallelism without NCCL.

    Every rank `publish`es its rows, sorted by destination, and a table of `world * segs_per_rank` row counts
    (destination rank major; for MoE one count per routed expert) in its arena; after a plane barrier `collect`
    copies the groups the peers hold for this rank, peers in rank order, with coalesced 16-byte loads over NVLink,
    and returns them with the peers' counts for this rank (what an all-to-all of the count table would deliver).
    `exchange` = barrier, publish, barrier, collect.  The reverse exchange (gradients, or the combine step) is the
    same call with the received counts as the table: its result comes back in the original send order.
    Replaces the padded-capacity all-to-alls of the reference (src/models/moe_expert_parallel.py:283-321)."""

    def __init__(self, plane: P2PPlane, max_rows: int, row_elems: int, dtype, segs_per_rank: int):
        self.plane, self.max_rows, self.d, self.dtype, self.spr = plane, int(max_rows), int(row_elems), dtype, int(segs_per_rank)
        esize = torch.empty(0, dtype=dtype).element_size()
        if (row_elems * esize) % 16 != 0:
            raise ValueError("row size must be a multiple of 16 bytes")
        self.row_bytes = row_elems * esize
        w = plane.world
        self.buf = plane.alloc(self.max_rows * self.d, dtype).view(self.max_rows, self.d)
        self.tab = plane.alloc(2 * w + w * self.spr, torch.int32)
        self._buf_ptrs = plane.peer_ptrs(self.buf)
        self._tab_ptrs = plane.peer_ptrs(self.tab)

    @staticmethod
    def arena_bytes(max_rows: int, row_elems: int, dtype, world: int, segs_per_rank: int) -> int:
        esize = torch.empty(0, dtype=dtype).element_size()
        return max_rows * row_elems * esize + 4 * (2 * world + world * segs_per_rank) + 4 * ALIGN

    def publish(self, rows: torch.Tensor, seg_counts: torch.Tensor):
        """rows [n, d] sorted by destination; seg_counts [world * segs_per_rank] integer tensor on the device."""
        n, w = rows.shape[0], self.plane.world
        if n > self.max_rows:
            raise RuntimeError(f"P2PAllToAll: {n} rows exceed the buffer of {self.max_rows}")
        if n:
            self.buf[:n].copy_(rows)
        c = seg_counts.to(torch.int32).view(w, self.spr)
        per_rank = c.sum(1, dtype=torch.int32)
        first = (torch.cumsum(per_rank, 0) - per_rank).to(torch.int32)
        self.tab.copy_(torch.cat([first, per_rank, c.reshape(-1)]))

    def collect(self, expect_rows=None):
        """-> (rows [m, d], counts [world * segs_per_rank] int32).  `expect_rows` (known in the reverse direction)
        saves the host read of the counts."""
        lib, w = _lib.lib(), self.plane.world
        counts = torch.empty(w * self.spr, dtype=torch.int32, device=self.plane.device)
        status = _lib.status_buffer(self.plane.device).data_ptr()
        if expect_rows is None or expect_rows == 0:      # counts only (also when nothing is to be copied)
            _lib.check_rc(lib.adana_p2p_all_to_all_pull(self._buf_ptrs, self._tab_ptrs, self.plane.rank, w, self.spr,
                                                        self.row_bytes, None, 0, counts.data_ptr(), status,
                                                        _lib.stream_ptr()), "adana_p2p_all_to_all_pull")
            if expect_rows is None:
                expect_rows = int(counts.sum().item())
        out = torch.empty((expect_rows, self.d), dtype=self.dtype, device=self.plane.device)
        if expect_rows:
            _lib.check_rc(lib.adana_p2p_all_to_all_pull(self._buf_ptrs, self._tab_ptrs, self.plane.rank, w, self.spr,
                                                        self.row_bytes, out.data_ptr(), expect_rows, counts.data_ptr(),
                                                        status, _lib.stream_ptr()), "adana_p2p_all_to_all_pull")
        return out, counts

    def exchange(self, rows: torch.Tensor, seg_counts: torch.Tensor, expect_rows=None):
        self.plane.barrier()          # nobody still reads what I published last time
        self.publish(rows, seg_counts)
        self.plane.barrier()          # every rank's rows and table are in place
        return self.collect(expect_rows)
