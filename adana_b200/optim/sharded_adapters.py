"""Every `--opt` name under the sharded engine.

The reference shards the model first (FSDP2) and then hands the DTensor parameters to whichever of its
optimizer classes was asked for (src/distributed/fsdp.py:105-116, src/main.py:74-253, 354-368).  The engine
keeps flat fp32 shards instead of DTensors, so the per-tensor classes of `adana_b200/optim/` get their
parameters in one of two ways:

`ShardViewOptimizer`  for optimizers whose update of an element needs only that element's own state and
    gradient plus scalars (AdamW, SGD, AdEMAMix, Lion, Signum, ADOPT, schedule-free, Sophia, Prodigy with
    its two all-reduced scalars).  The per-tensor class runs unchanged on 1-D views of this rank's piece of
    every parameter inside the engine's master / gradient shards: no communication, state sharded like
    the weights.

`OwnerOptimizer`  for optimizers that look at a whole tensor (Muon and Manau orthogonalise matrices, SOAP
    keeps eigenbases, Adafactor row / column moments, Lamb and MARS per-tensor norms).  Every parameter
    tensor has one owner rank (dealt by size, largest first, to the least loaded rank).  A step gathers each
    unit's reduced gradient, the owner steps its tensors with the unchanged per-tensor class on a full fp32
    copy it keeps, and one sum over the ranks (exactly one non-zero contributor per element) hands every
    rank its slice of the new values.  Results equal a one-process run of the same class.

Both scale the gradient by 1 / world (the engine reduces sums) and by the clip coefficient that
`Engine.grad_norm_and_clip` left on the device, and both leave the refresh of the bf16 compute weights to the
caller (`Engine.refresh_from_master`, which the training loop runs after any optimizer that is not the
engine's own).
"""
from __future__ import annotations

from typing import Callable, Dict, List

import torch
from torch import nn

ELEMENTWISE = {"adamw", "sgd", "ademamix", "ademamix-decaying-wd", "lion", "signsgd", "signum", "adopt", "sf-adamw",
               "sf-sgd", "sophiag", "prodigy"}
WHOLE_TENSOR = {"muon", "manau", "soap", "adafactor", "lamb", "mars"}


class _EngineAdapter(torch.optim.Optimizer):
    """Common part: an `torch.optim.Optimizer` whose `param_groups` ARE the inner optimizer's (LR schedulers and the
    logging code see the real hyper-parameters) and whose unknown attributes resolve on the inner optimizer
    (`train()` / `eval()` of the schedule-free classes, `update_hessian`, `update_last_grad`, ...)."""

    def __init__(self, engine, inner):
        super().__init__([nn.Parameter(torch.zeros(1, device=engine.device), requires_grad=False)], {})
        self.engine = engine
        self.inner = inner
        self.clip_pending = None
        self.defaults = inner.defaults
        self.param_groups = inner.param_groups      # the very same objects: what a scheduler sets, the inner class reads
        self.state = inner.state

    def __getattr__(self, name):
        if name in ("inner", "engine"):
            raise AttributeError(name)
        return getattr(self.inner, name)

    def zero_grad(self, set_to_none: bool = True):
        self.engine.zero_grad()

    def _grad_factor(self, clip: bool = True):
        eng = self.engine
        eng.finish_grad_sync()
        f = eng._clip[0] if (clip and eng.ecfg.grad_clip != 0.0 and self.clip_pending is not False) else None
        scale = 1.0 / eng.world if eng.world > 1 else 1.0
        return scale if f is None else f * scale

    def state_dict(self):
        return self.inner.state_dict()

    def load_state_dict(self, sd):
        self.inner.load_state_dict(sd)
        self.param_groups = self.inner.param_groups
        self.state = self.inner.state


class ShardViewOptimizer(_EngineAdapter):
    def __init__(self, engine, make_inner: Callable[[List[dict]], torch.optim.Optimizer], group_specs):
        self._pieces = []          # (parameter, unit, lo, hi) in local shard coordinates
        slot_of = {s.name: (u, s) for u in engine.units for s in u.layout.slots}
        specs = []
        for spec in group_specs:
            names = list(spec["param_names"] if "param_names" in spec else spec["params"])
            params, kept = [], []
            for n in names:
                u, s = slot_of[n]
                lo, hi = u.shard_off, u.shard_off + u.shard_len
                a, b = max(s.offset, lo), min(s.offset + s.numel, hi)
                if a >= b:
                    continue           # no element of this parameter lives on this rank
                p = nn.Parameter(u.master[a - lo:b - lo], requires_grad=True)   # shares the shard's storage
                self._pieces.append((p, u, a - lo, b - lo))
                params.append(p)
                kept.append(n)
            g = {k: v for k, v in spec.items() if k not in ("params", "param_names")}
            if not params:             # an optimizer group may not be empty: a zero-size stand-in keeps the group order
                params, kept = [nn.Parameter(torch.zeros(0, device=engine.device))], []
            g["params"], g["param_names"] = params, kept
            specs.append(g)
        super().__init__(engine, make_inner(specs))
        if engine.world > 1:
            for g in self.inner.param_groups:
                if "fsdp_in_use" in g:
                    g["fsdp_in_use"] = True    # Prodigy: all-reduce its two scalars (src/optim/prodigy.py:224-230)

    def _bind_grads(self, clip: bool = True):
        f = self._grad_factor(clip)
        for u in self.engine.units:
            u.grad_shard.mul_(f)
        for p, u, x0, x1 in self._pieces:
            p.grad = u.grad_shard[x0:x1]

    @torch.no_grad()
    def step(self, closure=None, **kw):
        self._bind_grads()
        out = self.inner.step(**kw) if kw else self.inner.step()
        self.clip_pending = None
        return out

    @torch.no_grad()
    def update_hessian(self, *a, **kw):      # Sophia: squares of the (sampled-label) gradient, element by element
        self._bind_grads(clip=False)
        return self.inner.update_hessian(*a, **kw)


class OwnerOptimizer(_EngineAdapter):
    def __init__(self, engine, make_inner: Callable[[List[dict]], torch.optim.Optimizer], group_specs):
        eng = engine
        self._slots = {s.name: (u, s) for u in eng.units for s in u.layout.slots}
        order = sorted(self._slots, key=lambda n: (-self._slots[n][1].numel, n))
        load = [0] * max(1, eng.world)
        self.owner: Dict[str, int] = {}
        for n in order:                       # largest first, to the least loaded rank: identical on every rank
            r = min(range(len(load)), key=lambda i: (load[i], i))
            self.owner[n] = r
            load[r] += self._slots[n][1].numel
        full = eng.full_param_dict("master")  # collective: every rank takes part, the owner keeps its tensors
        self._mine: Dict[str, nn.Parameter] = {}
        specs = []
        for spec in group_specs:
            names = list(spec["param_names"] if "param_names" in spec else spec["params"])
            params, kept = [], []
            for n in names:
                if self.owner[n] != eng.rank:
                    continue
                p = nn.Parameter(full[n].clone().float(), requires_grad=True)
                self._mine[n] = p
                params.append(p)
                kept.append(n)
            g = {k: v for k, v in spec.items() if k not in ("params", "param_names")}
            if not params:
                params, kept = [nn.Parameter(torch.zeros(0, device=eng.device))], []
            g["params"], g["param_names"] = params, kept
            specs.append(g)
        del full
        super().__init__(engine, make_inner(specs))
        if hasattr(self.inner, "world_size"):
            # a class that deals its matrices to the ranks itself (Muon's work partition with an all-reduce of the
            # updates, src/optim/muon.py:519-567) already holds only this rank's share here: it acts as one process
            self.inner.world_size, self.inner.rank = 1, 0

    def _bind_grads(self):
        f = self._grad_factor()
        eng = self.engine
        for u in eng.units:
            full = eng._gather_full(u.grad_shard, u)          # collective, unit by unit
            for s in u.layout.slots:
                p = self._mine.get(s.name)
                if p is not None:
                    p.grad = (full[s.offset:s.offset + s.numel].view(s.shape) * f).to(p.dtype)
            del full

    def _scatter_params(self):
        eng = self.engine
        for u in eng.units:
            if u.shard_len == u.padded:                        # not sharded: the owner is this rank
                for s in u.layout.slots:
                    u.master[s.offset:s.offset + s.numel].copy_(self._mine[s.name].detach().reshape(-1))
                continue
            flat = torch.zeros(u.padded, dtype=torch.float32, device=eng.device)
            for s in u.layout.slots:
                p = self._mine.get(s.name)
                if p is not None:
                    flat[s.offset:s.offset + s.numel].copy_(p.detach().reshape(-1))
            eng.comm.all_reduce_sum(flat)                      # one non-zero contributor per element: exact
            u.master.copy_(flat[u.shard_off:u.shard_off + u.shard_len])
            del flat

    @torch.no_grad()
    def step(self, closure=None, **kw):
        self._bind_grads()
        out = self.inner.step(**kw) if kw else self.inner.step()
        self._scatter_params()
        self.clip_pending = None
        return out

    @torch.no_grad()
    def update_last_grad(self, *a, **kw):     # MARS keeps the previous gradient of each of its tensors
        return self.inner.update_last_grad(*a, **kw)

    def load_state_dict(self, sd):
        super().load_state_dict(sd)
        # the owners' fp32 copies follow the engine's master weights (which a checkpoint load has just restored)
        full = self.engine.full_param_dict("master")
        with torch.no_grad():
            for n, p in self._mine.items():
                p.copy_(full[n])
