"""Learning-rate schedule factors (multipliers of the peak LR) as small callable objects.

Behaviour parity with the reference's schedule lambdas (src/optim/schedule.py:6-171):
`cos_inf` = linear warm-up from 1/div, cosine to 1/(div*final_div), then flat;
`wsd` = warm-up / hold / decay with six decay shapes; `powerlaw` = warm-up then
(1 + t/ts)^p clamped at a saturation value.  Each object is picklable, so a scheduler
built on it can be checkpointed, and exposes `table(n)` for vectorised evaluation.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np


class _Schedule:
    def __call__(self, step: int) -> float:  # pragma: no cover - interface
        raise NotImplementedError

    def table(self, n: int) -> np.ndarray:
        return np.array([self(i) for i in range(n)], dtype=np.float64)


def _warmup(step: int, n_warmup: int, div: float) -> float:
    f = step / n_warmup
    return f + (1.0 - f) / div


@dataclass
class CosInf(_Schedule):
    n_iterations: int
    n_warmup: int
    div_factor: float
    final_div_factor: float
    n_inf: int = 0

    def __call__(self, step: int) -> float:
        floor = 1.0 / self.div_factor / self.final_div_factor
        n_anneal = self.n_iterations - self.n_inf
        if step < self.n_warmup:
            return _warmup(step, self.n_warmup, self.div_factor)
        if step < n_anneal:
            t = (step - self.n_warmup) / (n_anneal - self.n_warmup)
            return floor + 0.5 * (1.0 - floor) * (1.0 + math.cos(math.pi * t))
        return floor


_DECAY_SHAPES = {
    "linear": lambda x, f: f + (1 - f) * (1 - x),
    "exp": lambda x, f: f ** x,
    "cosine": lambda x, f: f + (1 - f) * 0.5 * (1 + math.cos(math.pi * x)),
    "square": lambda x, f: f + (1 - f) * (1 - x * x),
    "sqrt": lambda x, f: f + (1 - f) * (1 - math.sqrt(x)),
}
_DECAY_SHAPES["miror_cosine"] = lambda x, f: 2 * _DECAY_SHAPES["linear"](x, f) - _DECAY_SHAPES["cosine"](x, f)


@dataclass
class WSD(_Schedule):
    n_iterations: int
    final_lr_factor: float = 0.0
    n_warmup: int = 1000
    init_div_factor: float = 100
    fract_decay: float = 0.1
    decay_type: str = "linear"

    def __post_init__(self):
        if self.decay_type not in _DECAY_SHAPES:
            raise ValueError(f"decay type {self.decay_type} is not in {sorted(_DECAY_SHAPES)}")

    def __call__(self, step: int) -> float:
        n_decay = int(self.fract_decay * self.n_iterations)
        n_hold = self.n_iterations - n_decay
        if step < self.n_warmup:
            return _warmup(step, self.n_warmup, self.init_div_factor)
        if step < n_hold:
            return 1.0
        if step < self.n_iterations:
            return _DECAY_SHAPES[self.decay_type]((step - n_hold) / n_decay, self.final_lr_factor)
        return self.final_lr_factor


@dataclass
class PowerLaw(_Schedule):
    n_iterations: int
    n_warmup: int
    init_value: float = 1.0
    saturation_value: float = 0.0
    power: float = -0.5
    time_scale: float = 1.0

    def __call__(self, step: int) -> float:
        if step < self.n_warmup:
            return (step / self.n_warmup) * self.init_value
        v = self.init_value * (1.0 + (step - self.n_warmup) / self.time_scale) ** self.power
        return max(v, self.saturation_value) if self.power < 0 else min(v, self.saturation_value)


# function-style constructors with the reference's names
def cos_inf_schedule(n_iterations, n_warmup, div_factor, final_div_factor, n_inf):
    return CosInf(n_iterations, n_warmup, div_factor, final_div_factor, n_inf)


def wsd_schedule(n_iterations, final_lr_factor=0.0, n_warmup=1000, init_div_factor=100,
                 fract_decay=0.1, decay_type="linear"):
    return WSD(n_iterations, final_lr_factor, n_warmup, init_div_factor, fract_decay, decay_type)


def powerlaw_schedule_with_warmup(n_iterations, n_warmup, init_value=1.0, saturation_value=0.0,
                                  power=-0.5, time_scale=1.0):
    return PowerLaw(n_iterations, n_warmup, init_value, saturation_value, power, time_scale)


def build_scheduler(args, opt):
    """Scheduler factory keyed by `--scheduler` (reference: src/main.py:387-455)."""
    import torch

    name = args.scheduler
    if name == "none":
        return None
    if name in ("cos", "linear"):
        max_lr = [g.get("lr", args.lr) for g in opt.param_groups]
        return torch.optim.lr_scheduler.OneCycleLR(
            optimizer=opt, max_lr=max_lr, total_steps=args.iterations,
            pct_start=args.warmup_steps / args.iterations, anneal_strategy=name,
            cycle_momentum=False, div_factor=1e2, final_div_factor=args.final_div_factor)
    if name == "cos_inf":
        lam = CosInf(args.iterations, args.warmup_steps, args.div_factor, args.final_div_factor,
                     args.cos_inf_steps)
    elif name == "wsd":
        lam = WSD(args.iterations, args.wsd_final_lr_scale, args.warmup_steps, 1e2,
                  args.wsd_fract_decay, args.decay_type)
    elif name == "powerlaw":
        lam = PowerLaw(args.iterations, args.warmup_steps, args.powerlaw_init_value,
                       args.powerlaw_saturation_value, args.powerlaw_power, args.powerlaw_time_scale)
    else:
        raise NotImplementedError(f"Unknown scheduler type: {name}.")
    return torch.optim.lr_scheduler.LambdaLR(opt, lam)
