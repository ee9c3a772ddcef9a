"""Per-layer / per-neuron training-dynamics statistics around optimizer steps.

Capability parity with the reference's `DynamicsLogger` (src/logger/logger.py:12-573, configuration
src/logger/rotational_logger.yaml): every `interval` optimizer steps the parameters are snapshotted before the
step, and after it a configurable set of statistics is computed per parameter:

    matrices (dim >= 2; a "neuron" is a row):  {layer,neuron}_norm, _grad_norm, _update_norm, _relative_update,
        _angular_update, _grad_alignment, _grad_velocity_alignment, _mean_second_grad_moment,
        _second_grad_moment_std_mean_ratio, _scaled_grad_norm, _scaled_grad_wd_projection
    vectors / scalars:                         scalar_rms, scalar_update_rms, scalar_grad_rms

Buffered values are written as appended pickles to `<output_folder>/dynamics.pkl` (down-sampled in time with an
RMS reducer, at most `disk_max_channels` neurons per layer) and/or as wandb scalars / histograms.

The design differs from the reference in two ways.  The statistics are a table (`STATS`: name -> function of a
`_Snapshot`), so a new statistic is one entry.  And the logger reads state through a *source*: a plain
`nn.Module` + `torch.optim.Optimizer` pair (`ModuleSource`) or the kernel engine (`EngineSource`), whose flat
sharded buffers are gathered into named full tensors — under a sharded engine every rank constructs the logger
(the gathers are collectives) and only the rank with `write=True` computes and stores statistics.
"""
from __future__ import annotations

import copy
import pickle
import types
from collections import defaultdict
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Dict, Optional

import torch
import torch.nn.functional as F
import yaml

DEFAULT_CFG = {
    "interval": 5,
    "stats": ["layer_norm", "neuron_norm", "layer_grad_norm", "neuron_grad_norm", "layer_update_norm",
              "neuron_update_norm", "layer_angular_update", "neuron_angular_update", "layer_relative_update",
              "neuron_relative_update", "scalar_rms", "scalar_update_rms", "scalar_grad_rms"],
    "disk_save_interval": None, "disk_stats": "all", "disk_max_channels": 16, "disk_downsample": 10,
    "wandb_interval": 5, "wandb_stats": "all",
}


def load_logger_config(path: Optional[str]) -> dict:
    cfg = copy.deepcopy(DEFAULT_CFG)
    if path:
        with open(path) as f:
            cfg.update(yaml.safe_load(f) or {})
    return cfg


# ---- where parameters, gradients and optimizer moments come from -----------------------------------------------
class ModuleSource:
    collective = False

    def __init__(self, model, optimizer):
        self.model, self.optimizer = model, optimizer

    def params(self):
        return {n: p.detach().clone() for n, p in self.model.named_parameters()}

    def grads(self):
        return {n: (p.grad.detach().clone() if p.grad is not None else None) for n, p in self.model.named_parameters()}

    def moments(self, which):
        keys = {"m": ("exp_avg", "m", "dana_m", "adamw_exp_avg"), "v": ("exp_avg_sq", "v", "dana_v", "adamw_exp_avg_sq")}[which]
        out = {}
        for n, p in self.model.named_parameters():
            st = self.optimizer.state.get(p, {})
            for k in keys:
                if k in st and torch.is_tensor(st[k]):
                    out[n] = st[k].detach().clone()
                    break
        return out


class EngineSource:
    def __init__(self, engine):
        self.engine = engine
        self.collective = engine.sharded and engine.world > 1

    def params(self):
        return self.engine.full_param_dict("master")

    def grads(self):
        scale = 1.0 / self.engine.world
        return {k: v * scale for k, v in self.engine.full_param_dict("grad").items()}

    def moments(self, which):
        return self.engine.full_param_dict(which)


# ---- statistics --------------------------------------------------------------------------------------------------
@dataclass
class _Snapshot:
    pre: torch.Tensor
    post: torch.Tensor
    grad: Optional[torch.Tensor]
    m_pre: Optional[torch.Tensor]
    v_post: Optional[torch.Tensor]
    eps: float

    @property
    def diff(self):
        return self.post - self.pre

    @property
    def scaled_grad(self):
        return self.grad / (self.v_post.sqrt() + 1e-8)


def _rows(t):
    return t.flatten(1)


def _lnorm(t):
    return torch.linalg.vector_norm(t.flatten())


def _nnorm(t):
    return torch.linalg.vector_norm(_rows(t), dim=1)


def _lcos(a, b):
    return F.cosine_similarity(a.flatten(), b.flatten(), dim=0)


def _ncos(a, b):
    return F.cosine_similarity(_rows(a), _rows(b), dim=1)


def _angle(cos):
    return torch.acos(cos.clamp(-1, 1))


def _rms(t):
    return t.square().mean().sqrt()


def _needs(*fields):
    def deco(fn):
        fn.needs = fields
        return fn
    return deco


# name -> (applies to matrices?, function).  Functions return None when their inputs are missing.
STATS: Dict[str, tuple] = {
    "layer_norm": (True, lambda s: _lnorm(s.pre)),
    "neuron_norm": (True, lambda s: _nnorm(s.pre)),
    "layer_grad_norm": (True, _needs("grad")(lambda s: _lnorm(s.grad))),
    "neuron_grad_norm": (True, _needs("grad")(lambda s: _nnorm(s.grad))),
    "layer_update_norm": (True, lambda s: _lnorm(s.diff)),
    "neuron_update_norm": (True, lambda s: _nnorm(s.diff)),
    "layer_relative_update": (True, lambda s: (_lnorm(s.diff) + s.eps) / (_lnorm(s.pre) + s.eps)),
    "neuron_relative_update": (True, lambda s: (_nnorm(s.diff) + s.eps) / (_nnorm(s.pre) + s.eps)),
    # angles are computed in float64: small rotations drown in fp32 rounding
    "layer_angular_update": (True, lambda s: _angle(_lcos(s.pre.double(), s.post.double()))),
    "neuron_angular_update": (True, lambda s: _angle(_ncos(s.pre.double(), s.post.double()))),
    "layer_grad_alignment": (True, _needs("grad")(lambda s: _lcos(s.grad, s.pre))),
    "neuron_grad_alignment": (True, _needs("grad")(lambda s: _ncos(s.grad, s.pre))),
    "layer_grad_velocity_alignment": (True, _needs("grad")(
        lambda s: _lcos(s.grad, s.m_pre) if s.m_pre is not None else torch.zeros((), device=s.pre.device))),
    "neuron_grad_velocity_alignment": (True, _needs("grad")(
        lambda s: _ncos(s.grad, s.m_pre) if s.m_pre is not None else torch.zeros(s.pre.shape[0], device=s.pre.device))),
    "layer_mean_second_grad_moment": (True, _needs("v_post")(lambda s: s.v_post.mean())),
    "neuron_mean_second_grad_moment": (True, _needs("v_post")(lambda s: _rows(s.v_post).mean(dim=1))),
    "layer_second_grad_moment_std_mean_ratio": (True, _needs("v_post")(lambda s: s.v_post.flatten().std() / s.v_post.mean())),
    "neuron_second_grad_moment_std_mean_ratio": (True, _needs("v_post")(
        lambda s: _rows(s.v_post).std(dim=1) / _rows(s.v_post).mean(dim=1))),
    "layer_scaled_grad_norm": (True, _needs("grad", "v_post")(lambda s: _lnorm(s.scaled_grad))),
    "neuron_scaled_grad_norm": (True, _needs("grad", "v_post")(lambda s: _nnorm(s.scaled_grad))),
    "layer_scaled_grad_wd_projection": (True, _needs("grad", "v_post")(
        lambda s: (s.pre.flatten() * s.scaled_grad.flatten()).sum() / _lnorm(s.pre).square())),
    "neuron_scaled_grad_wd_projection": (True, _needs("grad", "v_post")(
        lambda s: (_rows(s.pre) * _rows(s.scaled_grad)).sum(dim=1) / _nnorm(s.pre).square())),
    "scalar_rms": (False, lambda s: _rms(s.pre)),
    "scalar_update_rms": (False, lambda s: _rms(s.diff)),
    "scalar_grad_rms": (False, _needs("grad")(lambda s: _rms(s.grad))),
}

REDUCERS = defaultdict(lambda: "rms")        # every current statistic is non-negative or is logged as a magnitude


def _reduce(values: torch.Tensor, how: str, dim: int):
    if how == "mean":
        return values.mean(dim=dim)
    if how == "rms":
        return values.square().mean(dim=dim).sqrt()
    if how == "first":
        return values.select(dim, 0)
    raise ValueError(f"unknown reducer {how}")


class DynamicsLogger:
    def __init__(self, model, optimizer, cfg, output_folder, wandb=False, source=None, write=True):
        self.model, self.optimizer = model, optimizer
        self.iteration = 0
        self.output_folder = output_folder
        self.wandb = wandb
        self.write = write
        self.cfg = {**copy.deepcopy(DEFAULT_CFG), **copy.deepcopy(cfg)}
        for key in ("disk_stats", "wandb_stats"):
            if self.cfg[key] == "all":
                self.cfg[key] = list(self.cfg["stats"])
        unknown = set(self.cfg["stats"]) - set(STATS)
        if unknown:
            raise ValueError(f"unknown dynamics statistics: {sorted(unknown)}")
        if source is None:
            engine = getattr(model, "_engine", None) or getattr(optimizer, "engine", None)
            source = EngineSource(engine) if engine is not None else ModuleSource(model, optimizer)
        self.source = source
        self.stats = defaultdict(lambda: defaultdict(list))
        self.interval = self._interval_at(0)
        self._wandb_ready = False
        # the optimizer's own step stays reachable as `original_step`; LR schedulers that wrap `step` later see ours
        optimizer.original_step = optimizer.step
        logger = self

        def stepped(opt_self, *a, **k):
            return logger.step(*a, **k)

        optimizer.step = types.MethodType(stepped, optimizer)

    def _interval_at(self, it):
        spec = self.cfg["interval"]
        if isinstance(spec, int):
            return spec
        cur = spec[0][1]
        for start, every in spec:          # [(iter0, interval0), (iter1, interval1), ...] with iter0 < iter1 < ...
            if start <= it:
                cur = every
        return cur

    # -----------------------------------------------------------------------------------------------------------
    def step(self, *args, **kwargs):
        self.interval = self._interval_at(self.iteration)
        eps = self.optimizer.defaults.get("eps", 1e-8)
        if self.iteration % self.interval != 0:
            out = self.optimizer.original_step(*args, **kwargs)
            self.iteration += 1
            return out
        need_v = any("second_grad_moment" in s or "scaled_grad" in s for s in self.cfg["stats"])
        need_m = any("velocity" in s for s in self.cfg["stats"])
        pre = self.source.params()
        grads = self.source.grads()
        m_pre = self.source.moments("m") if need_m else {}
        out = self.optimizer.original_step(*args, **kwargs)
        post = self.source.params()
        v_post = self.source.moments("v") if need_v else {}
        if self.write:
            self._compute(pre, post, grads, m_pre, v_post, eps)
            self._maybe_flush()
        self.iteration += 1
        return out

    @torch.no_grad()
    def _compute(self, pre, post, grads, m_pre, v_post, eps):
        for name, p0 in pre.items():
            snap = _Snapshot(p0, post[name], grads.get(name), m_pre.get(name), v_post.get(name), eps)
            is_matrix = p0.dim() >= 2
            for stat in self.cfg["stats"]:
                for_matrix, fn = STATS[stat]
                if for_matrix != is_matrix:
                    continue
                if any(getattr(snap, f) is None for f in getattr(fn, "needs", ())):
                    continue
                val = fn(snap)      # angles are computed and kept in double (small angles drown in fp32 noise)
                self.stats[stat][name].append(val if val.dtype == torch.float64 else val.float())

    def _maybe_flush(self):
        t_disk = self.cfg["disk_save_interval"] or 0
        t_wandb = self.cfg["wandb_interval"] or 0
        if t_disk and (self.iteration + self.interval) % (t_disk * self.interval) == 0:
            self.log_to_disk()
        if self.wandb and t_wandb and (self.iteration + self.interval) % (t_wandb * self.interval) == 0:
            self.log_to_wandb()

    # -----------------------------------------------------------------------------------------------------------
    def log_to_disk(self, free_buffers=True):
        t_disk = self.cfg["disk_save_interval"]
        ds = self.cfg["disk_downsample"]
        out = {}
        for stat in self.cfg["disk_stats"]:
            out[stat] = {}
            for pname, values in self.stats[stat].items():
                v = torch.stack(values[-t_disk:])
                if self.cfg["disk_max_channels"] > 0 and v.dim() > 1:
                    v = v[:, :self.cfg["disk_max_channels"]]
                if ds > 1:
                    if t_disk % ds:
                        raise ValueError("disk_save_interval must be a multiple of disk_downsample")
                    v = _reduce(v.reshape(t_disk // ds, ds, -1), REDUCERS[stat], 1)
                out[stat][pname] = v.cpu()
        path = Path(self.output_folder)
        path.mkdir(parents=True, exist_ok=True)
        with open(path / "dynamics.pkl", "ab") as f:       # one pickle per flush, appended
            pickle.dump(out, f)
        if free_buffers:
            self.free_buffers("disk")

    def log_to_wandb(self, free_buffers=True):
        import wandb

        t_wandb = self.cfg["wandb_interval"]
        out = {}
        for stat in self.cfg["wandb_stats"]:
            for pname, values in self.stats[stat].items():
                v = _reduce(torch.stack(values[-t_wandb:]), REDUCERS[stat], 0).cpu().numpy()
                out[f"{stat}/{pname}"] = wandb.Histogram(v) if v.size > 1 else v
        if not self._wandb_ready:
            wandb.define_metric("iter")
            for k in out:
                wandb.define_metric(k, step_metric="iter")
            self._wandb_ready = True
        out["iter"] = self.iteration - (t_wandb - 1) * self.interval
        wandb.log(data=out)
        if free_buffers:
            self.free_buffers("wandb")

    def free_buffers(self, set_name="all"):
        """Drop values every consumer (disk, wandb) has already taken."""
        if set_name == "all":
            self.stats.clear()
            return
        main, other = {"disk": ("disk_stats", "wandb_stats"), "wandb": ("wandb_stats", "disk_stats")}[set_name]
        other_active = bool(self.cfg["wandb_interval"] and self.wandb) if other == "wandb_stats" else bool(self.cfg["disk_save_interval"])
        keep = max(self.cfg["disk_save_interval"] or 0, self.cfg["wandb_interval"] or 0)
        for stat in self.cfg[main]:
            if stat in self.cfg[other] and other_active:
                for pname in self.stats[stat]:
                    self.stats[stat][pname] = self.stats[stat][pname][-keep:]
            else:
                self.stats.pop(stat, None)

    @staticmethod
    def load_stats(path):
        """Concatenate the appended pickles of a `dynamics.pkl` into {stat: {param: tensor[time, ...]}}."""
        frags = []
        with open(path, "rb") as f:
            while True:
                try:
                    frags.append(pickle.load(f))
                except EOFError:
                    break
        return {stat: {p: torch.cat([fr[stat][p] for fr in frags]) for p in frags[0][stat]} for stat in frags[0]}
