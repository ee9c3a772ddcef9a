"""The log-time momentum family: ADana, Dana-MK4, Dana-Star, Dana-Star-MK4.

One pure elementwise update (`logtime_update_`) serves four users: the per-tensor
`torch.optim.Optimizer` classes below (CPU, oracle and DDP paths), the flat-shard update
of the sharded engine (`adana_b200/runtime/engine.py`), the CUDA kernel's numerics tests,
and Manau's non-matrix parameters.

Update rule per element, with t the 1-based step of the parameter, alpha = delta/(delta+t),
lr the scheduled learning rate of the group and sched = lr / lr_peak:

    m   <- lerp(m, g, alpha)                       v <- (1-alpha) v + alpha g^2
    ADana / Dana-MK4:
        n    = 1 / (sqrt(v) + eps)
        af   = (1+t)^(1-kappa) * |m| n             (clipped at `clipsnr` for MK4)
        p   <- p - lr g n - lr gamma3 (sign(m) af + m n)
    Dana-Star / Dana-Star-MK4 (tau = running estimate of how often a coordinate is "on"):
        tau <- lerp(tau, |g| / (|g| + sqrt(v) + eps), alpha)
        r    = max(min(tau,1/2)/(1-min(tau,1/2)), 1/(1+t))
        n    = sqrt(r) / (sqrt(v) + eps)
        af   = max(tau t, 1)^(1-kappa) * |m| n / r (clipped at `clipsnr` for MK4)
        p   <- p - lr g n - lr gamma3 sign(m) (r af + |m| n)
    then  p <- p (1 - wd sched / (1 + t/wd_ts))    (or (1 - wd sched) without decaying WD)

Weight decay is independent of the peak LR.  Parity: reference src/optim/adana.py:82-153 and
src/optim/dana_star_mk4.py:105-205; state-dict keys (`step, m, v, tau` and the logged scalars,
group keys `lr, delta, epsilon, weight_decay, weighted_step_count`) follow those classes so
that checkpoints are interchangeable.
"""
from __future__ import annotations

from typing import Iterable, Optional

import torch
from torch.optim import Optimizer


def wd_multiplier(wd: float, sched: float, step: int, wd_decaying: bool, wd_ts: float) -> float:
    """The factor every parameter is multiplied by after the update step."""
    if wd_decaying:
        return 1.0 - wd / (1.0 + step / wd_ts) * sched
    return 1.0 - wd * sched


@torch.no_grad()
def logtime_update_(p, g, m, v, tau, *, lr: float, alpha: float, step: int, kappa: float,
                    clipsnr: Optional[float], eps: float, gamma3: float, wd_mult: float,
                    diagnostics: bool = False):
    """In-place update of (p, m, v[, tau]) from gradient g; `tau is None` selects ADana."""
    m.lerp_(g, alpha)
    v.mul_(1.0 - alpha).addcmul_(g, g, value=alpha)
    denom = torch.sqrt(v).add_(eps)
    expo = 1.0 - kappa
    if tau is None:
        norm = 1.0 / denom
        mfac = m.abs() * norm
        af = (1.0 + step) ** expo * mfac
        if clipsnr is not None:
            af = af.clamp(max=clipsnr)
        long_term = torch.sign(m) * af + m * norm
    else:
        ag = g.abs()
        tau.lerp_(ag / (ag + denom), alpha)
        ct = tau.clamp(max=0.5)
        floor = 1.0 / (1.0 + step)
        reg = floor + torch.relu(ct / (1.0 - ct) - floor)
        eff_t = (tau * step).clamp(min=1.0)
        norm = torch.sqrt(reg) / denom
        mn = m.abs() * norm
        mfac = mn / reg
        af = eff_t ** expo * mfac
        if clipsnr is not None:
            af = af.clamp(max=clipsnr)
        long_term = torch.sign(m) * (reg * af + mn)
    upd = (-lr) * g * norm + (-lr) * gamma3 * long_term
    p.add_(upd)
    p.mul_(wd_mult)
    if diagnostics:
        return {"current_alpha": af.mean(), "gradient_norm": g.norm(),
                "auto_factor_mean": mfac.mean(), "m_norm": m.norm()}
    return None


class _LogTimeBase(Optimizer):
    _has_tau = False

    def __init__(self, params: Iterable, lr=1.0, delta=8.0, kappa=1.0, epsilon=1e-8,
                 weight_decay=0.0, clipsnr=None, wd_decaying=False, wd_ts=1.0,
                 gamma_3_factor=1.0, use_foreach=False, diagnostics=True):
        defaults = dict(lr=lr, delta=delta, epsilon=epsilon, weight_decay=weight_decay,
                        weighted_step_count=0)
        self.lr = lr
        self.delta = delta
        self.kappa = kappa
        self.epsilon = epsilon
        self.weight_decay = weight_decay
        self.clipsnr = clipsnr
        self.wd_decaying = wd_decaying
        self.wd_ts = wd_ts
        self.gamma_3_factor = gamma_3_factor
        self.use_foreach = use_foreach
        self.diagnostics = diagnostics
        super().__init__(params, defaults)

    def _init_state(self, p, state):
        state["step"] = 0
        state["m"] = torch.zeros_like(p)
        state["v"] = torch.zeros_like(p)
        if self._has_tau:
            state["tau"] = torch.zeros_like(p)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            lr = group["lr"]
            sched = lr / self.lr
            group["weighted_step_count"] += sched
            delta, wd, eps = group["delta"], group["weight_decay"], group["epsilon"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self.state[p]
                if len(state) == 0:
                    self._init_state(p, state)
                state["step"] += 1
                t = state["step"]
                diag = logtime_update_(
                    p, p.grad, state["m"], state["v"], state.get("tau") if self._has_tau else None,
                    lr=lr, alpha=delta / (delta + t), step=t, kappa=self.kappa,
                    clipsnr=self.clipsnr, eps=eps, gamma3=self.gamma_3_factor,
                    wd_mult=wd_multiplier(wd, sched, t, self.wd_decaying, self.wd_ts),
                    diagnostics=self.diagnostics)
                if diag is not None:
                    # on sharded (DTensor) parameters a norm or mean comes back as a pending cross-rank reduction;
                    # the logged scalars are stored reduced, as plain tensors, so that the state can be checkpointed
                    diag = {k: (v.full_tensor() if hasattr(v, "full_tensor") else v) for k, v in diag.items()}
                    state["current_alpha"] = diag["current_alpha"]
                    state["gradient_norm"] = diag["gradient_norm"]
                    state["auto_factor_mean"] = diag["auto_factor_mean"]
                    state["current_kappa_factor"] = diag["current_alpha"] / diag["auto_factor_mean"]
                    state["m_norm"] = diag["m_norm"]
        return loss


class ADana(_LogTimeBase):
    """`--opt adana` (clipsnr=None) and `--opt dana-mk4` (clipsnr=c)."""
    _has_tau = False


class DanaStarMK4(_LogTimeBase):
    """`--opt dana-star` (clipsnr=None) and `--opt dana-star-mk4` (clipsnr=c)."""
    _has_tau = True

    def __init__(self, params, lr=1.0, delta=8.0, kappa=1.0, mk4A=0.0, mk4B=0.0, epsilon=1e-8,
                 weight_decay=0.0, clipsnr=1.0, weight_time=False, wd_decaying=False, wd_ts=1.0,
                 gamma_3_factor=1.0, use_foreach=False, diagnostics=True):
        if mk4A != 0.0 or mk4B != 0.0 or weight_time:
            raise ValueError("mk4A, mk4B must be 0 and weight_time False (Manau carries the generalised form)")
        self.mk4A = 0.0
        self.mk4B = 0.0
        self.weight_time = False
        super().__init__(params, lr=lr, delta=delta, kappa=kappa, epsilon=epsilon,
                         weight_decay=weight_decay, clipsnr=clipsnr, wd_decaying=wd_decaying,
                         wd_ts=wd_ts, gamma_3_factor=gamma_3_factor, use_foreach=use_foreach,
                         diagnostics=diagnostics)


DANA_STAR_MK4 = DanaStarMK4  # the reference's class name
