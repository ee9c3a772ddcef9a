"""Update rules of the ADana family and AdEMAMix as pure functions on NumPy arrays.

Each `*_rule(...)` returns a pair `(init, update)`:

    state = init(params)
    delta_params, state = update(grads, state, params)      # params <- params + lr * delta_params

in the style of a gradient transformation: the returned `delta_params` already carries the descent sign and
the additive weight-decay term `-wd * p`; `scale_by_learning_rate` multiplies by the (scheduled) outer rate.

Two time conventions exist for the same formulas, and the rules take `convention=`:

* ``"optax"`` — the reference's JAX statement (jax/optimizers.py:94-239, 242-410, 413-605): one shared counter
  starting at 0, EMA weight alpha = (1 + count/delta)^-1 (so the very first step has alpha = 1), effective
  time max(count, 1) in ADana / Dana-MK4 and max(tau*count, 1) in Dana-Star-MK4.
* ``"torch"`` — the reference's PyTorch classes (src/optim/adana.py:82-153, src/optim/dana_star_mk4.py:105-205):
  step t starting at 1, alpha = delta/(delta + t), ADana's time factor (1 + t)^(1-kappa), Dana-Star's
  max(tau*t, 1)^(1-kappa) with the 1/(1+t) floor on tau's odds.

With ``"torch"`` the rules reproduce `adana_b200.optim.logtime` bit-for-bit in float64 up to rounding, which is
what the tests check; weight decay in that convention is still additive here (the classes use a
multiplicative, LR-independent decay), so comparisons are made with `wd=None`.
"""
from __future__ import annotations

from typing import Callable, NamedTuple, Optional, Union

import numpy as np

Schedule = Callable[[float], float]
ScalarOrSchedule = Union[float, Schedule]


def powerlaw_schedule(init_value: float, saturation_value: float, power: float, time_scale: float) -> Schedule:
    """t -> max(init * (1 + t/time_scale)^power, saturation)."""
    return lambda t: np.maximum(init_value * (1.0 + t / time_scale) ** power, saturation_value)


def _sched(x: Optional[ScalarOrSchedule], default=0.0) -> Schedule:
    if x is None:
        return lambda t: default
    return x if callable(x) else (lambda t: x)


class LogTimeState(NamedTuple):
    count: int
    m: np.ndarray
    v: np.ndarray
    tau: Optional[np.ndarray]


def _clock(count: int, delta: float, convention: str):
    """-> (t used in formulas, EMA weight alpha)."""
    if convention == "optax":
        return float(count), 1.0 / (1.0 + count / delta)
    if convention == "torch":
        t = count + 1
        return float(t), delta / (delta + t)
    raise ValueError(f"unknown convention {convention}")


def _logtime_rule(g2, g3, delta, eps, kappa, clipsnr, wd, with_tau, convention):
    g2, g3, wd = _sched(g2, 1.0), _sched(g3, 1.0), _sched(wd, 0.0)

    def init(params):
        z = np.zeros_like(params, dtype=np.float64)
        return LogTimeState(0, z.copy(), z.copy(), z.copy() if with_tau else None)

    def update(grads, state, params=None):
        u = np.asarray(grads, dtype=np.float64)
        t, alpha = _clock(state.count, delta, convention)
        v = state.v * (1 - alpha) + alpha * u * u
        m = state.m * (1 - alpha) + alpha * u
        root = np.sqrt(v) + eps
        if with_tau:
            tau = state.tau * (1 - alpha) + alpha * np.abs(u) / (np.abs(u) + root)
            odds = np.minimum(tau, 0.5)
            odds = odds / (1.0 - odds)
            reg = np.maximum(odds, 1.0 / (1.0 + t))
            eff = np.maximum(tau * t, 1.0)
            norm = np.sqrt(reg) / root
        else:
            tau, reg = None, 1.0
            eff = max(t, 1.0) if convention == "optax" else 1.0 + t
            norm = 1.0 / root
        m_norm = np.abs(m) * norm
        af = eff ** (1.0 - kappa) * m_norm / reg
        if clipsnr is not None:
            af = np.minimum(af, clipsnr)
        time_for_g = eff if convention == "optax" else t
        out = -g2(time_for_g) * u * norm - g3(time_for_g) * np.sign(m) * (reg * af + m_norm)
        if params is not None:
            out = out - wd(state.count) * np.asarray(params, dtype=np.float64)
        return out, LogTimeState(state.count + 1, m, v, tau)

    return init, update


def adana_rule(g2=1.0, g3=1.0, delta=8.0, epsilon=1e-8, kappa=1.0, wd=None, convention="optax"):
    """ADana: log-time EMAs, sign-momentum term scaled by t^(1-kappa) |m|/sqrt(v), no SNR clipping."""
    return _logtime_rule(g2, g3, delta, epsilon, kappa, None, wd, False, convention)


def dana_mk4_rule(g2=1.0, g3=1.0, delta=8.0, epsilon=1e-8, kappa=1.0, clipsnr=2.0, wd=None, convention="optax"):
    """Dana-MK4: ADana with the momentum factor clipped at `clipsnr`."""
    return _logtime_rule(g2, g3, delta, epsilon, kappa, clipsnr, wd, False, convention)


def dana_star_mk4_rule(g2=1.0, g3=1.0, delta=8.0, epsilon=1e-8, kappa=1.0, clipsnr=2.0, wd=None,
                       convention="optax"):
    """Dana-Star-MK4: per-coordinate activity estimate tau rescales both the step and the effective time."""
    return _logtime_rule(g2, g3, delta, epsilon, kappa, clipsnr, wd, True, convention)


def dana_star_rule(g2_constant: float, g3_constant: float, kappa: float, epsilon: float = 1e-8, clipsnr: float = 2.0,
                   beta_time_scale: float = 6.0, wd: Optional[ScalarOrSchedule] = None):
    """The first Dana-Star ("galaxy", jax/optimizers.py:69-85, 607-758), which the m-sweeps compare MK4 against.  Per
    coordinate, with beta = (1 + count / 6)^-1 for all three averages and t = count:
        v, m, tau EMAs as in MK4 (tau from |u| / (|u| + sqrt(v) + eps) with the NEW v)
        reg = max(min(tau, 1/2) / (1 - min(tau, 1/2)), 1 / (1 + t)),  r = sqrt(reg),  eff = max(tau t, 1)
        update = -g2 u (r / (sqrt v + eps)) min(1, clipsnr sqrt(v) / (r |u| + eps))  -  g3(eff) m r / (sqrt v + eps)
    g3(x) = g3_constant (1 + x)^(1 - kappa) is read at each coordinate's own effective time: where MK4 clips the
    momentum's size, this rule clips the gradient term."""
    wd = _sched(wd, 0.0)
    g3 = powerlaw_schedule(g3_constant, 0.0, 1.0 - kappa, 1.0)

    def init(params):
        z = np.zeros_like(params, dtype=np.float64)
        return LogTimeState(0, z.copy(), z.copy(), z.copy())

    def update(grads, state, params=None):
        u = np.asarray(grads, dtype=np.float64)
        t = float(state.count)
        beta = 1.0 / (1.0 + t / beta_time_scale)
        v = state.v * (1 - beta) + beta * u * u
        tau = state.tau * (1 - beta) + beta * np.abs(u) / (np.abs(u) + np.sqrt(v) + epsilon)
        m = state.m * (1 - beta) + beta * u
        half = np.minimum(tau, 0.5)
        r = np.sqrt(np.maximum(half / (1.0 - half), 1.0 / (1.0 + t)))
        eff = np.maximum(tau * t, 1.0)
        root = np.sqrt(v)
        scale = r / (root + epsilon)
        out = -g2_constant * u * scale * np.minimum(1.0, clipsnr * root / (r * np.abs(u) + epsilon)) - g3(eff) * m * scale
        if params is not None:
            out = out - wd(state.count) * np.asarray(params, dtype=np.float64)
        return out, LogTimeState(state.count + 1, m, v, tau)

    return init, update


class AdEMAMixState(NamedTuple):
    count: int
    fast: Optional[np.ndarray]
    slow: np.ndarray
    sq: np.ndarray


def ademamix_rule(beta1=0.9, beta2=0.999, beta3=0.9999, alpha=2.0, gamma_3_factor=1.0, epsilon=1e-8, wd=None):
    """AdEMAMix (reference jax/optimizers.py:761-992): fast EMA (bias-corrected) + alpha * slow EMA over a
    bias-corrected second moment; beta1 = 0 uses the raw gradient as the fast term.  Every hyper-parameter may
    be a schedule of the step count."""
    b1, b2, b3 = _sched(beta1), _sched(beta2), _sched(beta3)
    al, g3f, wd = _sched(alpha), _sched(gamma_3_factor), _sched(wd, 0.0)
    use_fast = not (np.isscalar(beta1) and beta1 == 0)

    def init(params):
        z = np.zeros_like(params, dtype=np.float64)
        return AdEMAMixState(0, z.copy() if use_fast else None, z.copy(), z.copy())

    def update(grads, state, params=None):
        u = np.asarray(grads, dtype=np.float64)
        c = state.count
        step = c + 1
        bc2 = 1.0 - b2(c) ** step
        slow = state.slow * b3(c) + (1 - b3(c)) * u
        sq = state.sq * b2(c) + (1 - b2(c)) * u * u
        denom = np.sqrt(sq) / np.sqrt(bc2) + epsilon
        if use_fast:
            fast = state.fast * b1(c) + (1 - b1(c)) * u
            lead = fast / (1.0 - b1(c) ** step)
        else:
            fast, lead = None, u
        out = (lead + al(c) * g3f(c) * slow) / denom
        if params is not None:
            out = out + wd(c) * np.asarray(params, dtype=np.float64)
        return -out, AdEMAMixState(step, fast, slow, sq)

    return init, update


def scale_by_learning_rate(rule, learning_rate: ScalarOrSchedule):
    """Chain a rule with an outer learning rate (scalar or schedule of the step count)."""
    init, update = rule
    lr = _sched(learning_rate)

    def scaled(grads, state, params=None):
        out, new = update(grads, state, params)
        return lr(state.count) * out, new

    return init, scaled
