"""Moonlight-style distributed Muon on the engine's flat rank shards: gather → Newton–Schulz → scatter.

The reference's `DistributedMuon` under FSDP2 (src/optim/muon.py:126-440) leaves every matmul of the
Newton–Schulz chain to DTensor, which redistributes operands per product.  Here the chain is moved as a
whole, one unit (transformer block) at a time:

  1. shard-local, elementwise: momentum  buf <- mu*buf + g ; ns_in = g + mu*buf (Nesterov), cast to bf16;
  2. ONE bf16 all-gather of the unit's `ns_in` shards (half the bytes of an fp32 gradient gather);
  3. the unit's matrices are dealt round-robin to the ranks; a rank orthogonalises its matrices with the
     three-GEMM tcgen05 chain (`adana_b200/ops/muon_ns.py`) and writes them into a zeroed bf16 unit buffer;
  4. ONE bf16 reduce-scatter-sum of that buffer hands each rank its flat slice of every update (each element
     has exactly one non-zero contributor, so the sum is exact);
  5. shard-local: p <- p(1 - lr*wd) - lr*0.2*sqrt(max(A,B)) * update, per parameter slot.

Vectors, embeddings and the LM head (2-D with >= 10000 rows) take the Muon codebases' AdamW shard-locally.
Gradient averaging over ranks and the clip coefficient left on the device by `Engine.grad_norm_and_clip`
are folded into step 1.  State (`muon_buffer`, `adamw_exp_avg`, `adamw_exp_avg_sq`) is flat per unit and
sharded like the master weights; `state_dict()` returns these flat shards keyed by unit name.
"""
from __future__ import annotations

import math

import torch
from torch import nn

from ..optim.muon import orthogonalize
from .comm import wait


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
        self.plan = []
        k = 0
        for u in engine.units:
            mats, rest = [], []
            for s in u.layout.slots:
                if len(s.shape) >= 2 and s.shape[0] < 10000:
                    mats.append((s, k % engine.world if engine.sharded else 0))
                    k += 1
                else:
                    rest.append(s)
            self.plan.append((u, mats, rest))

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
