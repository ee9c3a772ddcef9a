"""Adam-type baselines used for ablations: AdamW with (decaying) independent weight decay,
AdEMAMix and AdEMAMix with (decaying) independent weight decay.

Parity: reference src/optim/adamw_decaying_wd.py:5-86, src/optim/ademamix.py:11-195,
src/optim/ademamix_decaying_wd.py:25-190.  State keys are the reference's
(`exp_avg, exp_avg_sq` / `exp_avg_fast, exp_avg_slow, exp_avg_sq`, `step`).
"""
from __future__ import annotations

import math

import torch
from torch.optim import Optimizer

from .logtime import wd_multiplier


def linear_warmup_scheduler(step, alpha_end, alpha_start=0.0, warmup=1):
    if step >= warmup:
        return alpha_end
    a = step / float(warmup)
    return (1.0 - a) * alpha_start + a * alpha_end


def linear_hl_warmup_scheduler(step, beta_end, beta_start=0.0, warmup=1):
    """Warm beta up so that the EMA half-life grows linearly."""
    if step >= warmup:
        return beta_end

    def half_life(beta, eps=1e-8):
        return math.log(0.5) / math.log(beta + eps) - 1

    a = step / float(warmup)
    hl = (1.0 - a) * half_life(beta_start) + a * half_life(beta_end)
    return math.pow(0.5, 1.0 / (hl + 1.0))


class AdamWDecayingWD(Optimizer):
    """Bias-corrected Adam step followed by p *= 1 - wd*sched/(1 + t/wd_ts)."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), epsilon=1e-8, weight_decay=0.0,
                 wd_decaying=False, wd_ts=1.0):
        self.initial_lr = lr
        self.wd_decaying = wd_decaying
        self.wd_ts = wd_ts
        super().__init__(params, dict(lr=lr, betas=betas, epsilon=epsilon, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            lr = group["lr"]
            sched = lr / self.initial_lr
            b1, b2 = group["betas"]
            eps, wd = group["epsilon"], group["weight_decay"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p)
                    st["exp_avg_sq"] = torch.zeros_like(p)
                st["step"] += 1
                t = st["step"]
                st["exp_avg"].mul_(b1).add_(g, alpha=1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
                bc1, bc2 = 1 - b1 ** t, 1 - b2 ** t
                denom = (st["exp_avg_sq"].sqrt() / bc2 ** 0.5).add_(eps)
                p.addcdiv_(st["exp_avg"], denom, value=-lr / bc1)
                if wd != 0:
                    p.mul_(wd_multiplier(wd, sched, t, self.wd_decaying, self.wd_ts))
        return loss


class AdEMAMix(Optimizer):
    """Mixture of a fast and a slow gradient EMA over an Adam second moment; coupled WD."""

    _independent_wd = False

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999, 0.9999), alpha=2.0, beta3_warmup=None,
                 alpha_warmup=None, eps=1e-8, weight_decay=0, gamma_3_factor=1.0,
                 wd_decaying=False, wd_ts=1.0):
        if lr < 0 or eps < 0 or weight_decay < 0 or alpha < 0:
            raise ValueError("lr, eps, weight_decay and alpha must be non-negative")
        for i, b in enumerate(betas):
            if not 0.0 <= b < 1.0:
                raise ValueError(f"Invalid beta parameter at index {i}: {b}")
        defaults = dict(lr=lr, betas=betas, eps=eps, alpha=alpha, beta3_warmup=beta3_warmup,
                        alpha_warmup=alpha_warmup, weight_decay=weight_decay,
                        gamma_3_factor=gamma_3_factor)
        if self._independent_wd:
            defaults.update(wd_decaying=wd_decaying, wd_ts=wd_ts)
        self.initial_lr = lr
        super().__init__(params, defaults)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            lr, wd, eps = group["lr"], group["weight_decay"], group["eps"]
            b1, b2, b3_final = group["betas"]
            sched = lr / self.initial_lr
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad
                if g.is_sparse:
                    raise RuntimeError("AdEMAMix does not support sparse gradients.")
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg_fast"] = torch.zeros_like(p) if b1 != 0.0 else None
                    st["exp_avg_slow"] = torch.zeros_like(p)
                    st["exp_avg_sq"] = torch.zeros_like(p)
                st["step"] += 1
                t = st["step"]
                bc1, bc2 = 1 - b1 ** t, 1 - b2 ** t
                alpha = group["alpha"]
                if group["alpha_warmup"] is not None:
                    alpha = linear_warmup_scheduler(t, alpha_end=alpha, alpha_start=0,
                                                    warmup=group["alpha_warmup"])
                b3 = b3_final
                if group["beta3_warmup"] is not None:
                    b3 = linear_hl_warmup_scheduler(t, beta_end=b3_final, beta_start=b1,
                                                    warmup=group["beta3_warmup"])
                st["current_alpha"] = alpha
                st["current_beta3"] = b3
                st["current_one_minus_beta3"] = 1 - b3
                if b1 != 0.0:
                    fast = st["exp_avg_fast"].mul_(b1).add_(g, alpha=1 - b1)
                else:
                    fast = g
                st["exp_avg_slow"].mul_(b3).add_(g, alpha=1 - b3)
                st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
                denom = (st["exp_avg_sq"].sqrt() / math.sqrt(bc2)).add_(eps)
                update = (fast.div(bc1) + alpha * st["exp_avg_slow"] * group["gamma_3_factor"]) / denom
                if self._independent_wd:
                    # the decay multiplies the parameter before the step is applied
                    p.mul_(wd_multiplier(wd, sched, t, group["wd_decaying"], group["wd_ts"]))
                    p.add_(update, alpha=-lr)
                else:
                    update.add_(p, alpha=wd)
                    p.add_(update, alpha=-lr)
        return loss


class AdEMAMixDecayingWD(AdEMAMix):
    """AdEMAMix whose weight decay is independent of the peak LR and may decay as 1/(1+t/ts)."""

    _independent_wd = True


AdEMAMix_DecayingWD = AdEMAMixDecayingWD  # the reference's class name
