"""Risk dynamics of momentum SGD ("Dana") on a quadratic, solved by implicit Euler in log-time.

For every Hessian eigenvalue lambda_j the second moments (rho_j, sigma_j, chi_j) — squared parameter error,
squared momentum, and their cross term in that eigen-direction — obey a linear 3x3 system driven by the
total risk, with time-dependent coefficients built from the schedules g1 (gradient into momentum), g2
(gradient into parameters), g3 (momentum into parameters) and delta (momentum decay):

    d/dt (rho, sigma, chi)_j = Omega_j(t) (rho, sigma, chi)_j + Gamma(t) lambda_j * (2 risk(t))
    2 risk(t) = 2 risk_inf + sum_j lambda_j rho_j(t)

Substituting s = log(1 + t) and taking one backward-Euler step of size ds gives, per mode, a 3x3 solve;
the coupling through the risk is a rank-one term handled in closed form (Sherman–Morrison), so a step is
O(d).  Same scheme and coefficients as the reference's `ode_resolvent_log_implicit` (jax/dana_plrf.py:58-278);
here the per-mode systems are one batched `numpy.linalg.solve` instead of a hand-expanded inverse, and the loop
is plain NumPy.  `adaptive` divides g3 ('adam') or g1 ('rmsprop_dana') by sqrt(2 risk) as a stand-in for the
gradient norm.  Returns times t and TWICE the risk, as in the paper's plots.

Options of the schedule experiments (jax/kappa_sweep_plot.py:76-222, dynamical_schedule_plot.py:68-200,
danastar_schedule_plot.py:70-222):
  momentum=True          also return sum_j sigma_j, the squared momentum norm ||y||^2, at every time
  risk_renormalized      "DanaStar" scaling: g2 and g3 are divided by sqrt(2 risk) at every step
  dynamic_g3="ratio"     g3(t) is multiplied by min(2 risk / (2 ||y||^2), 1): momentum is trusted only while the risk
                         is larger than the momentum's energy
  dynamic_g3="inv_sqrt_risk"   g3(t) is divided by sqrt(2 risk) (on top of `risk_renormalized`, if that is set)
  dynamic_g3=(A, B, k0)  g3(t) is multiplied by (2 risk)^A (||y||^2)^B (1+t)^k0 clipped to [1, 1+t]: a kappa
                         schedule read off the trajectory
  shifted_clock          g1, g2 and delta are read at t + 1 and g3 at t, as those scripts do
"""
from __future__ import annotations

from typing import Callable, NamedTuple, Optional

import numpy as np


class DanaHparams(NamedTuple):
    g1: Callable[[float], float]
    g2: Callable[[float], float]
    g3: Callable[[float], float]
    delta: Callable[[float], float]


class ODEInputs(NamedTuple):
    eigs_K: np.ndarray
    rho_init: np.ndarray
    chi_init: np.ndarray
    sigma_init: np.ndarray
    risk_infinity: float


def _coefficients(lam, g1, g2, g3, dl, batch, approximate):
    """-> Omega [d,3,3] (rows/cols ordered rho, sigma, chi) and Gamma [3]."""
    d = lam.shape[0]
    one = np.ones(d)
    om = np.empty((d, 3, 3))
    if approximate:
        om[:, 0, 0] = -2 * g2 * lam
        om[:, 0, 1] = 0.0
        om[:, 0, 2] = -2 * g3 * one
        om[:, 1, 0] = 0.0
        om[:, 1, 1] = -2 * dl * one
        om[:, 1, 2] = 2 * g1 * lam
        om[:, 2, 0] = g1 * lam
        om[:, 2, 1] = -g3 * one
        om[:, 2, 2] = -dl - g2 * lam
        gamma = np.array([g2 ** 2, g1 ** 2, 0.0]) / batch
        return om, gamma
    bb = (batch + 1.0) / batch
    eff = g2 + g1 * g3                      # total gradient coefficient reaching the parameters in one step
    om[:, 0, 0] = -2 * eff * lam + bb * eff ** 2 * lam ** 2
    om[:, 0, 1] = g3 ** 2 * (1 - dl) ** 2 * one
    om[:, 0, 2] = -2 * g3 * (1 - dl) + 2 * g3 * eff * (1 - dl) * lam
    om[:, 1, 0] = bb * g1 ** 2 * lam ** 2
    om[:, 1, 1] = (dl ** 2 - 2 * dl) * one
    om[:, 1, 2] = 2 * g1 * (1 - dl) * lam
    om[:, 2, 0] = g1 * lam - bb * g1 * eff * lam ** 2
    om[:, 2, 1] = -g3 * (1 - dl) ** 2 * one
    om[:, 2, 2] = -dl - (g2 * (1 - dl) + 2 * (1 - dl) * g1 * g3) * lam
    gamma = np.array([eff ** 2, g1 ** 2, -g1 * eff]) / batch
    return om, gamma


def solve_risk_ode(inputs: ODEInputs, hp: DanaHparams, batch: int, t_max: float, dt: float = 1e-2,
                   approximate: bool = False, adaptive: Optional[str] = None, momentum: bool = False,
                   risk_renormalized: bool = False, dynamic_g3=None, shifted_clock: bool = False):
    lam = np.asarray(inputs.eigs_K, dtype=np.float64)
    state = np.stack([inputs.rho_init, inputs.sigma_init, inputs.chi_init], axis=1).astype(np.float64)  # [d,3]
    two_r_inf = 2.0 * inputs.risk_infinity
    s_grid = np.arange(0.0, np.log(t_max), dt)
    two_risk = two_r_inf + float(lam @ state[:, 0])
    out = np.empty(len(s_grid))
    mom_out = np.empty(len(s_grid))
    mom = float(state[:, 1].sum())
    eye = np.eye(3)[None]
    for i, s in enumerate(s_grid):
        out[i] = two_risk
        mom_out[i] = mom
        clock = np.exp(s + dt)             # d t / d s at the end of the step
        t = clock - 1.0
        ts = clock if shifted_clock else t
        gn = np.sqrt(two_risk) if adaptive else 1.0
        g1 = hp.g1(ts) / (gn if adaptive == "rmsprop_dana" else 1.0)
        g3 = hp.g3(t) / (gn if adaptive == "adam" else 1.0)
        g2 = hp.g2(ts)
        if dynamic_g3 == "ratio":
            g3 *= min(two_risk / (2.0 * mom + 1e-10), 1.0)
        elif dynamic_g3 == "inv_sqrt_risk":
            g3 /= np.sqrt(two_risk)
        elif dynamic_g3 is not None:
            pa, pb, k0 = dynamic_g3
            m_eff = mom if mom != 0.0 else 1.0
            g3 *= min(max(two_risk ** pa * m_eff ** pb * np.exp(k0 * s), 1.0), np.exp(s))
        if risk_renormalized:
            scale = 1.0 / np.sqrt(two_risk + 1e-10)
            g2, g3 = g2 * scale, g3 * scale
        om, gamma = _coefficients(lam, g1, g2, g3, hp.delta(ts), batch, approximate)
        h = dt * clock
        A = eye - h * om                                              # [d,3,3]
        force = gamma[None, :] * lam[:, None]                         # [d,3]
        rhs = np.stack([state + h * two_r_inf * force, force], axis=2)    # two right-hand sides per mode
        sol = np.linalg.solve(A, rhs)
        x, y = sol[:, :, 0], sol[:, :, 1]
        # the risk couples the modes through sum_j lambda_j rho_j: rank-one correction in closed form
        coupling = h * float(lam @ x[:, 0]) / (1.0 - h * float(lam @ y[:, 0]))
        state = x + coupling * y
        two_risk = two_r_inf + float(lam @ state[:, 0])
        mom = float(state[:, 1].sum())
    if momentum:
        return np.exp(s_grid) - 1.0, out, mom_out
    return np.exp(s_grid) - 1.0, out
