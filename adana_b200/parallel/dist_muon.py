"""Moonlight-style distributed Muon on the engine's flat rank shards: gather -> Newton-Schulz -> scatter.

The reference's `DistributedMuon` under FSDP2 (src/optim/muon.py:126-440) leaves every matmul of the
Newton-Schulz chain to DTensor, which redistributes operands per product.  Here the chain is moved as a whole.

Kernel chain (GPU; one rank, replicated weights, or rank shards on the peer-memory plane; csrc/muon_chain.cu):

  1. `muon_momentum`, shard-local, every unit: buf <- mu*buf + g, ns_in = g + mu*buf (Nesterov) rounded to bf16 into
     this rank's part of a symmetric staging buffer (the unit's gradient buffer, idle once the gradients are reduced),
     with partial sums of squares per matrix; then one "staged" flag per unit to every rank;
  2. every matrix has ONE owner rank, dealt by Newton-Schulz cost (largest first to the least loaded rank).  The owner
     pulls exactly its matrices' pieces out of the peers' staging buffers, scaled to unit Frobenius norm in the same
     pass (`muon_pull`, which waits - bounded - for the unit's flags), runs the 3-GEMM tcgen05 iteration with no
     transpose in memory (`ops/muon_ns.py::ns_chain`), and stores the result straight into the staging buffers of
     the ranks that hold those elements (`muon_push`); a "pushed" flag per unit follows its last matrix;
  3. `muon_apply`, shard-local, waits for the owners' flags: p <- p(1 - lr*wd) - lr*0.2*sqrt(max(A,B)) * update for
     matrix pieces, the Muon codebases' AdamW for vectors, embeddings and the LM head (2-D with >= 10000 rows), and
     stores the new bf16 weights into every rank's resident weight buffer.

Only the bytes of a rank's own matrices cross NVLink (once in, once out, bf16), no buffer is zero-padded and nothing
between the momentum update and the new weights runs as a PyTorch op.

Fallback (CPU / Gloo / NCCL without the plane / fp32 compute): the same five steps with torch ops, one bf16 all-gather
and one bf16 reduce-scatter-sum of a unit buffer that is zero except for this rank's matrices.

Gradient averaging over ranks and the clip coefficient left on the device by `Engine.grad_norm_and_clip` are folded
into step 1.  State (`muon_buffer`, `adamw_exp_avg`, `adamw_exp_avg_sq`) is flat per unit and sharded like the master
weights; `state_dict()` returns these flat shards keyed by unit name.
"""
from __future__ import annotations

import ctypes
import math
import os

import numpy as np
import torch
from torch import nn

from ..ops import _lib
from ..optim.muon import orthogonalize
from .comm import wait

MUON_FLAG_STAGED = 2048       # flag slots (8 per unit) of the two phases, above the gradient units' slots
MUON_FLAG_PUSHED = 4096
SEG_DTYPE = np.dtype([("a", "<i8"), ("b", "<i8"), ("kind", "<i4"), ("group", "<i4"), ("shape_factor", "<f4"),
                      ("mat", "<i4")])          # csrc/muon_chain.cu: struct Seg


def _u64(vals):
    return (ctypes.c_ulonglong * len(vals))(*[int(v) for v in vals])


def ns_cost(shape) -> int:
    """Multiply-adds of one Newton-Schulz iteration on a matrix: two products with the long side, one s x s square."""
    s_, l_ = min(shape), max(shape)
    return 2 * s_ * s_ * l_ + s_ ** 3


class ShardedMuon(torch.optim.Optimizer):
    def __init__(self, engine, args, group_specs):
        self.engine = engine
        self.lr = args.lr
        dev = engine.device
        groups = []
        for spec in group_specs:
            g = {"params": [nn.Parameter(torch.zeros(1, device=dev), requires_grad=False)],
                 "param_names": list(spec["param_names"] if "param_names" in spec else spec["params"])}
            if "weight_decay" in spec:
                g["weight_decay"] = spec["weight_decay"]
            groups.append(g)
        defaults = dict(lr=args.lr, weight_decay=args.weight_decay, momentum=getattr(args, "momentum", 0.95),
                        nesterov=bool(getattr(args, "nesterov", True)), ns_steps=getattr(args, "muon_ns_steps", 5),
                        matched_adamw_rms=getattr(args, "matched_adamw_rms", 0.2),
                        adamw_betas=(getattr(args, "beta1", 0.95), getattr(args, "beta2", 0.95)), adamw_eps=1e-8)
        super().__init__(groups, defaults)
        self.step_count = 0
        self.clip_pending = None
        # static plan: which slots are matrices, and who orthogonalises which
        found = []
        for ui, u in enumerate(engine.units):
            for s in u.layout.slots:
                if len(s.shape) >= 2 and s.shape[0] < 10000:
                    found.append((ns_cost((s.shape[0], math.prod(s.shape[1:]))), ui, s))
        n_owner = engine.world if (engine.sharded and engine.world > 1) else 1
        load = [0] * n_owner
        owner_of = {}
        for cost, ui, s in sorted(found, key=lambda c: (-c[0], c[1], c[2].offset)):
            r = min(range(n_owner), key=lambda i: (load[i], i))       # identical on every rank
            owner_of[(ui, s.name)] = r
            load[r] += cost
        self.plan = []
        for ui, u in enumerate(engine.units):
            mats = [(s, owner_of[(ui, s.name)]) for s in u.layout.slots if (ui, s.name) in owner_of]
            rest = [s for s in u.layout.slots if (ui, s.name) not in owner_of]
            self.plan.append((u, mats, rest))
        self.chain = None
        self._graphs = {}
        self._graph_ok = os.environ.get("ADANA_MUON_GRAPHS", "1") != "0"
        if self._chain_supported():
            self._setup_chain()

    # ---- kernel chain -------------------------------------------------------------------------------------------
    def _chain_supported(self) -> bool:
        eng = self.engine
        if eng.device.type != "cuda" or not _lib.available() or not _lib.has("adana_muon_apply"):
            return False
        if eng.cdt != torch.bfloat16:
            return False
        multi = eng.sharded and eng.world > 1
        if multi and (eng.plane is None or any(u.weights is None for u in eng.units)):
            return False
        for u, mats, _ in self.plan:
            if u.padded >= 2 ** 31 * 8:
                return False
            for s, _ in mats:
                if len(s.shape) != 2 or s.shape[0] % 8 or s.shape[1] % 8:
                    return False
        if multi and MUON_FLAG_STAGED + 8 * len(self.plan) > MUON_FLAG_PUSHED:
            return False
        return True

    def _setup_chain(self):
        eng = self.engine
        dev = eng.device
        multi = eng.sharded and eng.world > 1
        world = eng.world if multi else 1
        me = eng.rank if multi else 0
        parts_n = int(_lib.lib().adana_muon_parts())
        n_mats = sum(len(m) for _, m, _ in self.plan)
        rms = self.defaults["matched_adamw_rms"]
        units, mat_id = [], 0
        big, big_s = 8, 8
        for ui, (u, mats, rest) in enumerate(self.plan):
            lo, hi = u.shard_off, u.shard_off + u.shard_len
            rows, mine = [], []
            for s, owner in mats:
                a, b = max(s.offset, lo), min(s.offset + s.numel, hi)
                a, b = (a - lo, b - lo) if a < b else (0, 0)
                rows.append((a, b, 0, 0 if s.decay else 1, rms * math.sqrt(max(s.shape)), mat_id))
                if owner == me:
                    mine.append((s, mat_id))
                    big, big_s = max(big, s.numel), max(big_s, min(s.shape))
                mat_id += 1
            for s in rest:
                a, b = max(s.offset, lo), min(s.offset + s.numel, hi)
                if a < b:
                    rows.append((a - lo, b - lo, 1, 0 if s.decay else 1, 0.0, 0))
            table = np.array(rows, dtype=SEG_DTYPE) if rows else np.zeros(0, dtype=SEG_DTYPE)
            segs = torch.from_numpy(table.view(np.uint8).copy()).to(dev)
            units.append(dict(u=u, index=ui, segs=segs, n_segs=len(rows), n_mat_segs=len(mats), mine=mine,
                              max_len=max([r[1] - r[0] for r in rows], default=0)))
        bf = torch.bfloat16
        if multi:
            plane = eng.plane
            parts = plane.alloc(max(n_mats, 1) * parts_n, torch.float32)
            parts_ptrs = plane.peer_ptrs(parts)
            for d in units:
                u = d["u"]
                stage = u.grads.view(bf)        # 2 * padded bf16 elements of symmetric memory, idle during the optimizer phase
                d["ns"], d["upd"] = stage[:u.padded], stage[u.padded:2 * u.padded]
                d["ns_ptrs"], d["upd_ptrs"] = plane.peer_ptrs(d["ns"]), plane.peer_ptrs(d["upd"])
                d["w_ptrs"], d["n_dst"], d["push_off"] = plane.peer_ptrs(u.weights), world, u.shard_off
        else:
            parts = torch.zeros(max(n_mats, 1) * parts_n, dtype=torch.float32, device=dev)
            parts_ptrs = _u64([parts.data_ptr()])
            most = max(d["u"].padded for d in units)
            ns, upd = torch.empty(most, dtype=bf, device=dev), torch.empty(most, dtype=bf, device=dev)
            for d in units:
                u = d["u"]
                d["ns"], d["upd"] = ns[:u.padded], upd[:u.padded]
                d["ns_ptrs"], d["upd_ptrs"] = _u64([ns.data_ptr()]), _u64([upd.data_ptr()])
                push = u.low_precision and u.weights is not None
                d["w_ptrs"], d["n_dst"], d["push_off"] = (_u64([u.weights.data_ptr()]) if push else None), int(push), 0
        self.chain = dict(units=units, world=world, me=me, multi=multi, parts=parts, parts_ptrs=parts_ptrs,
                          X=torch.empty(big, dtype=bf, device=dev), Y=torch.empty(big, dtype=bf, device=dev),
                          A=torch.empty(big_s * big_s, dtype=bf, device=dev), B=torch.empty(big_s * big_s, dtype=bf, device=dev))

    def _ns_graphed(self, X, Y, A, B, steps: int):
        """The 3 * steps GEMM launches of one orthogonalisation, replayed from a CUDA graph per matrix shape (the
        workspace is fixed, so the captured pointers stay valid): small matrices are bound by launch rate otherwise.
        The first use of a shape runs eagerly, the second is captured; ADANA_MUON_GRAPHS=0 keeps everything eager."""
        from ..ops.muon_ns import ns_chain

        key = (tuple(X.shape), int(steps))
        g = self._graphs.get(key)
        if g is None or g == "eager":
            if g is None and self._graph_ok:
                self._graphs[key] = "warm"
            return ns_chain(X, Y, A, B, steps)
        if g == "warm":
            try:
                graph = torch.cuda.CUDAGraph()
                torch.cuda.synchronize(self.engine.device)
                with torch.cuda.graph(graph):
                    out = ns_chain(X, Y, A, B, steps)
                self._graphs[key] = g = (graph, out)
            except Exception:
                self._graphs[key] = "eager"
                return ns_chain(X, Y, A, B, steps)
        g[0].replay()
        return g[1]

    def _flags(self, base: int, unit_index: int) -> int:
        return self.engine.plane.base + 4 * (base + 8 * unit_index)

    @torch.no_grad()
    def _step_chain(self):
        from ..ops.muon_ns import ns_chain

        eng, ch = self.engine, self.chain
        lib = _lib.lib()
        g_decay, g_nodecay = self.param_groups[0], self.param_groups[1]
        mu, steps = g_decay["momentum"], g_decay["ns_steps"]
        self.step_count += 1
        t = self.step_count
        b1, b2 = g_decay["adamw_betas"]
        bias = (1 - b1 ** t) / math.sqrt(1 - b2 ** t)
        world, multi = ch["world"], ch["multi"]
        gscale = 1.0 / eng.world          # the engine reduces sums
        hyper = (ctypes.c_float * 9)(g_decay["lr"], g_nodecay["lr"], g_decay["weight_decay"], g_nodecay["weight_decay"],
                                     b1, b2, g_decay["adamw_eps"], bias, gscale)
        clip, stream = eng._clip.data_ptr(), _lib.stream_ptr()
        status = _lib.status_buffer(eng.device).data_ptr()
        plane = eng.plane if multi else None
        seq = t & 0xFFFFFFFF
        tmo = plane.timeout_ns if multi else 0
        if multi:
            plane.barrier()       # every rank's gradient reduction has finished reading the buffers staged into below
        def momentum(d):
            u = d["u"]
            u.ensure_state(["muon_buffer", "adamw_exp_avg", "adamw_exp_avg_sq"])
            if d["n_mat_segs"]:
                _lib.check_rc(lib.adana_muon_momentum(
                    u.grad_shard.data_ptr(), u.state["muon_buffer"].data_ptr(), d["ns"].data_ptr() + 2 * u.shard_off,
                    d["segs"].data_ptr(), d["n_mat_segs"], clip, gscale, float(mu), int(bool(g_decay["nesterov"])),
                    ch["parts"].data_ptr(), stream), "adana_muon_momentum")
            if multi:
                _lib.check_rc(lib.adana_p2p_signal(plane._flag_ptrs, plane.rank, world, MUON_FLAG_STAGED + 8 * d["index"],
                                                   seq, stream), "adana_p2p_signal")

        def orthogonalise(d):
            u = d["u"]
            for s, mat in d["mine"]:
                m, n = s.shape
                X, Y = ch["X"][:s.numel].view(m, n), ch["Y"][:s.numel].view(m, n)
                k = min(m, n)
                A, B = ch["A"][:k * k].view(k, k), ch["B"][:k * k].view(k, k)
                _lib.check_rc(lib.adana_muon_pull(
                    d["ns_ptrs"], ch["parts_ptrs"], world, u.shard_len, s.offset, s.numel, mat, 1e-7, X.data_ptr(),
                    self._flags(MUON_FLAG_STAGED, d["index"]) if multi else 0, seq, tmo, status, stream), "adana_muon_pull")
                out = self._ns_graphed(X, Y, A, B, steps)
                _lib.check_rc(lib.adana_muon_push(out.data_ptr(), d["upd_ptrs"], world, u.shard_len, s.offset, s.numel,
                                                  stream), "adana_muon_push")
            if multi:
                _lib.check_rc(lib.adana_p2p_signal(plane._flag_ptrs, plane.rank, world, MUON_FLAG_PUSHED + 8 * d["index"],
                                                   seq, stream), "adana_p2p_signal")

        def apply(d):
            u = d["u"]
            if d["n_segs"] == 0:
                return
            _lib.check_rc(lib.adana_muon_apply(
                u.master.data_ptr(), u.grad_shard.data_ptr(), d["upd"].data_ptr() + 2 * u.shard_off,
                u.state["adamw_exp_avg"].data_ptr(), u.state["adamw_exp_avg_sq"].data_ptr(), d["segs"].data_ptr(),
                d["n_segs"], hyper, clip, d["w_ptrs"], d["n_dst"], d["push_off"], d["max_len"],
                self._flags(MUON_FLAG_PUSHED, d["index"]) if multi else 0, seq, world, tmo, status, stream),
                "adana_muon_apply")

        if multi:
            # phase by phase over all units: a rank never waits for a peer while it still has work that peers wait for
            for phase in (momentum, orthogonalise, apply):
                for d in ch["units"]:
                    phase(d)
        else:
            # one staging buffer serves all units: unit by unit
            for d in ch["units"]:
                momentum(d)
                orthogonalise(d)
                apply(d)
        if multi:
            eng._sync_small()      # exact fp32 norm weights to every rank; ends with the barrier that completes the pushes

    @staticmethod
    def _overlap(slot, lo, hi):
        a, b = max(slot.offset, lo), min(slot.offset + slot.numel, hi)
        return (a, b) if a < b else None

    @torch.no_grad()
    def step(self, closure=None):
        eng = self.engine
        eng.finish_grad_sync()
        if eng.ecfg.grad_clip == 0.0 or self.clip_pending is False:
            eng._clip[0] = 1.0
        if self.chain is not None:
            self._step_chain()
            if (eng.plane or eng.ar_plane) is not None:
                eng._sumsq.zero_()
            eng.opt_step_count += 1
            eng.micro_step = 0
            self.clip_pending = None
            return None
        g_decay, g_nodecay = self.param_groups[0], self.param_groups[1]
        lr, mu = g_decay["lr"], g_decay["momentum"]
        self.step_count += 1
        t = self.step_count
        b1, b2 = g_decay["adamw_betas"]
        eps = g_decay["adamw_eps"]
        bias = (1 - b1 ** t) / math.sqrt(1 - b2 ** t)
        gscale = eng._clip[0] / eng.world
        sharded = eng.sharded and eng.world > 1
        for u, mats, rest in self.plan:
            u.ensure_state(["muon_buffer", "adamw_exp_avg", "adamw_exp_avg_sq"])
            lo, hi = u.shard_off, u.shard_off + u.shard_len
            g = u.grad_shard * gscale
            # 1. momentum on this rank's slice of every matrix
            ns_in = torch.zeros(u.shard_len, dtype=torch.bfloat16, device=g.device)
            for s, _ in mats:
                ov = self._overlap(s, lo, hi)
                if ov is None:
                    continue
                a, b = ov[0] - lo, ov[1] - lo
                buf = u.state["muon_buffer"][a:b].mul_(mu).add_(g[a:b])
                ns_in[a:b] = (g[a:b].add(buf, alpha=mu) if g_decay["nesterov"] else buf).to(torch.bfloat16)
            # 2. gather
            if sharded:
                full = torch.empty(u.padded, dtype=torch.bfloat16, device=g.device)
                wait(eng.comm.all_gather(ns_in, full))
            else:
                full = ns_in
            # 3. orthogonalise the matrices dealt to this rank
            upd_full = torch.zeros(u.padded, dtype=torch.bfloat16, device=g.device)
            for s, owner in mats:
                if owner != (eng.rank if sharded else 0):
                    continue
                M = full[s.offset:s.offset + s.numel].view(s.shape[0], -1)
                upd_full[s.offset:s.offset + s.numel] = orthogonalize(M, g_decay["ns_steps"]).reshape(-1)
            # 4. scatter
            if sharded:
                upd = torch.empty(u.shard_len, dtype=torch.bfloat16, device=g.device)
                wait(eng.comm.reduce_scatter_sum(upd_full, upd))
            else:
                upd = upd_full
            # 5. apply
            for s, _ in mats:
                ov = self._overlap(s, lo, hi)
                if ov is None:
                    continue
                a, b = ov[0] - lo, ov[1] - lo
                grp = g_decay if s.decay else g_nodecay
                A, B = s.shape[0], math.prod(s.shape[1:])
                adj = grp["lr"] * math.sqrt(max(A, B)) * grp["matched_adamw_rms"]
                u.master[a:b].mul_(1 - grp["lr"] * grp["weight_decay"]).add_(upd[a:b].float(), alpha=-adj)
            for s in rest:
                ov = self._overlap(s, lo, hi)
                if ov is None:
                    continue
                a, b = ov[0] - lo, ov[1] - lo
                grp = g_decay if s.decay else g_nodecay
                m1 = u.state["adamw_exp_avg"][a:b].lerp_(g[a:b], 1 - b1)
                m2 = u.state["adamw_exp_avg_sq"][a:b].lerp_(g[a:b].square(), 1 - b2)
                u.master[a:b].mul_(1 - grp["lr"] * grp["weight_decay"]).add_(m1 / (eps + m2.sqrt()), alpha=-grp["lr"] / bias)
        eng.refresh_from_master()
        if eng.plane is not None:
            eng._sumsq.zero_()
        eng.opt_step_count += 1
        eng.micro_step = 0
        self.clip_pending = None
        return None

    def zero_grad(self, set_to_none: bool = True):
        self.engine.zero_grad()

    # ---- checkpoint: flat shards keyed by unit ------------------------------------------------------------------
    def state_dict(self):
        groups = [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]
        state = {u.layout.name: {k: v.clone() for k, v in u.state.items()
                                 if k in ("muon_buffer", "adamw_exp_avg", "adamw_exp_avg_sq")}
                 for u, _, _ in self.plan}
        return {"state": state, "param_groups": groups, "step": self.step_count,
                "shard": {"rank": self.engine.rank, "world": self.engine.world}}

    def load_state_dict(self, sd):
        self.step_count = int(sd.get("step", 0))
        for g, saved in zip(self.param_groups, sd["param_groups"]):
            g.update({k: v for k, v in saved.items() if k != "params"})
        for u, _, _ in self.plan:
            for k, v in sd["state"].get(u.layout.name, {}).items():
                u.ensure_state([k])
                u.state[k].copy_(v.to(u.state[k].device))
