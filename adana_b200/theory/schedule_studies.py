"""Experiments on the risk ODE that motivate the long-momentum schedule g3(t) ~ (1+t)^-kappa of the ADana family.

All of them solve `theory.ode.solve_risk_ode` on the deterministic-equivalent spectrum of a power-law random-features
problem (eigenvalues j^-2alpha, weights from `deterministic.theory_rhos`, floor `theory_limit_loss`) with the schedules
g1 = 1 (or delta), g2 = lr constant, delta(t) = c / (c + t) with c = 4 + (alpha + beta) / alpha, and different g3:

  compare_optimizers   SGD (g3 = 0), Dana-constant (g3 = g g2 / d), Dana-decay (g3 = g g2 (1+t)^(-1/(2 alpha))) and
                       AdEMAMix written in the same variables (jax/plrf_ademamix_behavior.py:120-187)
  kappa_sweep          momentum as a running mean (g1 = delta) and g3 = c (1+t)^kappa growing, for a grid of kappa in
                       [0, 1), with the squared momentum norm tracked; at T = 10^k the exponents log R / log T and
                       log ||y||^2 / log T, the best kappa, and the kappa that the trajectory-driven schedule settles
                       at (jax/kappa_sweep_plot.py:229-520)
  crossing_kappa       momentum as a raw sum (g1 = 1) and g3 = (1+t)^kappa decaying, kappa in [-1.5, -0.2]: the kappa at
                       which (log R - log ||y||^2) / log T equals kappa, the self-consistent exponent;
                       `alpha_crossings` repeats it over alpha and fits it against 1 / (2 alpha)
                       (jax/alpha_sweep_crossing.py:174-340)
  dynamic_schedules    fixed g3 schedules against g3 = g2 min(R / ||y||^2, 1) (jax/dynamical_schedule_plot.py:207-420)
  danastar_schedules   the same comparison under the DanaStar division of g2 and g3 by sqrt(2R), with growing g3
                       schedules on a running-mean momentum (jax/danastar_schedule_plot.py:228-450); both report the
                       log-log slope of the late excess risk

    python -m adana_b200.theory.schedule_studies compare --alpha 1.5 --d 200 --out compare.json [--svg compare.svg]
    python -m adana_b200.theory.schedule_studies kappa-sweep --alpha 0.5 --d 300 --steps 1e5 --out sweep.json
    python -m adana_b200.theory.schedule_studies crossing --alphas 0.4 0.6 0.8 1.0 --out crossing.json
    python -m adana_b200.theory.schedule_studies dynamic --alpha 0.7 [--danastar] --out dynamic.json
"""
from __future__ import annotations

import argparse
import json
import math
from typing import Dict, Optional, Sequence

import numpy as np

from .deterministic import theory_limit_loss, theory_rhos
from .ode import DanaHparams, ODEInputs, solve_risk_ode
from .rules import powerlaw_schedule


def ode_inputs(alpha: float, beta: float, v: int, d: int) -> ODEInputs:
    eigs, rho = theory_rhos(alpha, beta, d)
    z = np.zeros_like(rho)
    return ODEInputs(eigs, rho, z, z.copy(), theory_limit_loss(alpha, beta, v, d))


def population_trace(alpha: float, v: int) -> float:
    return float(np.sum(np.arange(1, v + 1, dtype=np.float64) ** (-2.0 * alpha)))


def const(c: float):
    return powerlaw_schedule(c, 0.0, 0.0, 1)


def delta_schedule(alpha: float, beta: float, c: Optional[float] = None):
    return powerlaw_schedule(1.0, 0.0, -1.0, 4.0 + 2 * (alpha + beta) / (2 * alpha) if c is None else c)


def loglog_slope(t, y, t_from: float, t_to: float) -> float:
    m = (t >= t_from) & (t <= t_to) & (y > 0)
    return float(np.polyfit(np.log(t[m]), np.log(y[m]), 1)[0]) if m.sum() >= 2 else math.nan


def at_time(t, y, T: float) -> float:
    return float(y[int(np.argmin(np.abs(t - T)))])


# ---- SGD, Dana-constant, Dana-decay, AdEMAMix --------------------------------------------------------------------------
def compare_optimizers(alpha: float = 1.5, beta: float = 0.3, d: int = 500, v: Optional[int] = None, batch: int = 1,
                       steps: Optional[float] = None, lr_scale: float = 0.5, g2: float = 0.5, g3: float = 0.5,
                       delta: float = 8.0, dt: float = 1e-2, which: Sequence[str] = ("sgd", "dana-constant", "dana-decay", "ademamix")) -> Dict:
    v = 5 * d if v is None else v
    steps = float(d ** (2 * alpha)) if steps is None else steps
    inp = ode_inputs(alpha, beta, v, d)
    g2_base = lr_scale * min(1.0, batch / population_trace(alpha, v)) * g2
    G1, G2, Dl = const(1.0), const(g2_base), powerlaw_schedule(1.0, 0.0, -1.0, delta)
    hp = {}
    if "sgd" in which:
        hp["sgd"] = DanaHparams(G1, G2, const(0.0), Dl)
    if "dana-constant" in which:
        hp["dana-constant"] = DanaHparams(G1, G2, const(g3 * g2_base / d), Dl)
    if "dana-decay" in which:
        hp["dana-decay"] = DanaHparams(G1, G2, powerlaw_schedule(g3 * g2_base, 0.0, -1.0 / (2 * alpha), 1.0), Dl)
    if "ademamix" in which:
        T_mix = d ** alpha
        beta3_final, alpha_final = 1.0 - delta / T_mix, 0.5 * T_mix ** (1 - 1 / (2 * alpha))
        half_life = lambda b: math.log(0.5) / math.log(b + 1e-8) - 1

        def delta_mix(t):      # 1 - beta3(t) with AdEMAMix's half-life interpolation from 0.9 to beta3_final
            a = min(t / T_mix, 1.0)
            return 1.0 - 0.5 ** (1.0 / ((1 - a) * half_life(0.9) + a * half_life(beta3_final) + 1))

        hp["ademamix"] = DanaHparams(lambda t: 1.0 / (1.0 + t), G2, lambda t: g2_base * min(t / T_mix, 1.0) * alpha_final, delta_mix)
    out = {"args": dict(alpha=alpha, beta=beta, d=d, v=v, batch=batch, steps=steps, g2_base=g2_base, delta=delta),
           "risk_infinity": inp.risk_infinity, "runs": {}}
    for name, h in hp.items():
        t, two_r = solve_risk_ode(inp, h, batch, steps, dt)
        out["runs"][name] = {"t": t + 1, "loss": 0.5 * two_r}
    return out


# ---- kappa sweep -------------------------------------------------------------------------------------------------------
def kappa_sweep(alpha: float = 0.5, beta: float = 0.3, v: int = 2000, d: int = 500, batch: int = 1, steps: float = 1e6,
                dt: float = 1e-2, kappas: Optional[Sequence[float]] = None, powers=(0.0, 0.75, 1.0),
                risk_renormalized: bool = True, g1_is_delta: bool = True, g3_constant: Optional[float] = None) -> Dict:
    """`powers` = (A, B, base kappa) of the trajectory-driven schedule.  Returns curves, checkpoint tables at T = 10^k
    and, per checkpoint, the kappa of least risk and the effective kappa of the dynamic run."""
    kappas = np.linspace(0.0, 1.0, 30, endpoint=False) if kappas is None else np.asarray(kappas, dtype=np.float64)
    inp = ode_inputs(alpha, beta, v, d)
    c = 0.1 / math.sqrt(d) * 0.5 * min(1.0, batch / population_trace(alpha, v))
    Dl = delta_schedule(alpha, beta)
    G1 = Dl if g1_is_delta else const(1.0)
    g3c = c if g3_constant is None else g3_constant
    kw = dict(momentum=True, risk_renormalized=risk_renormalized, shifted_clock=True)
    runs = []
    for k in kappas:
        t, two_r, mom = solve_risk_ode(inp, DanaHparams(G1, const(c), powerlaw_schedule(g3c, 0.0, float(k), 1), Dl), batch, steps, dt, **kw)
        runs.append({"kappa": float(k), "t": t, "risk": 0.5 * two_r, "momentum": mom})
    t, two_r, mom = solve_risk_ode(inp, DanaHparams(G1, const(c), const(g3c), Dl), batch, steps, dt, dynamic_g3=tuple(powers), **kw)
    dyn = {"t": t, "risk": 0.5 * two_r, "momentum": mom}
    A, B, k0 = powers
    table = {}
    for e in range(1, int(math.floor(math.log10(steps))) + 1):
        T = 10.0 ** e
        R = np.array([at_time(r["t"], r["risk"], T) for r in runs])
        M = np.array([at_time(r["t"], r["momentum"], T) for r in runs])
        with np.errstate(divide="ignore", invalid="ignore"):
            eff = (A * math.log(2 * at_time(dyn["t"], dyn["risk"], T)) + B * math.log(max(at_time(dyn["t"], dyn["momentum"], T), 1e-300))) / math.log(T)
            table[int(T)] = {"risk": R, "momentum": M, "risk_exponent": np.log(R) / math.log(T),
                             "momentum_exponent": np.log(M) / math.log(T),
                             "heuristic": (A * np.log(R) + B * np.log(M)) / math.log(T) + k0,
                             "best_kappa": float(kappas[int(np.argmin(R))]),
                             "effective_kappa": float(min(max(eff + k0, 0.0), 1.0))}
    return {"args": dict(alpha=alpha, beta=beta, v=v, d=d, batch=batch, steps=steps, powers=list(powers)),
            "kappas": kappas, "runs": runs, "dynamic": dyn, "checkpoints": table}


def crossing_kappa(alpha: float, beta: float = 0.5, v: int = 4000, d: int = 1000, batch: int = 1, steps: float = 1e7,
                   target_T: Optional[float] = None, dt: float = 1e-2, kappas: Optional[Sequence[float]] = None):
    """-> (kappa where (log R - log ||y||^2) / log T = kappa at T = target_T, or None; the kappa grid; the ratio on it).
    Here g1 = 1 and g3 = (1+t)^kappa carry no learning-rate constant, and nothing is renormalised by the risk; a run
    that diverges (possible at the slow end of the grid) leaves NaN in the ratio and is skipped."""
    kappas = np.linspace(-1.5, -0.2, 30, endpoint=False) if kappas is None else np.asarray(kappas, dtype=np.float64)
    T = steps / 10 if target_T is None else target_T
    inp = ode_inputs(alpha, beta, v, d)
    c = 0.1 / math.sqrt(d) * 0.5 * min(1.0, batch / population_trace(alpha, v))
    Dl = delta_schedule(alpha, beta)
    ratio = []
    for k in kappas:
        t, two_r, mom = solve_risk_ode(inp, DanaHparams(const(1.0), const(c), powerlaw_schedule(1.0, 0.0, float(k), 1), Dl),
                                       batch, steps, dt, momentum=True, shifted_clock=True)
        R, M = 0.5 * at_time(t, two_r, T), at_time(t, mom, T)
        ratio.append((math.log(R) - math.log(M)) / math.log(T) if R > 0 and M > 0 else math.nan)
    ratio = np.array(ratio)
    diff = ratio - kappas
    for i in range(len(kappas) - 1):
        if np.isfinite(diff[i]) and np.isfinite(diff[i + 1]) and np.sign(diff[i]) != np.sign(diff[i + 1]):
            return float(kappas[i] - diff[i] * (kappas[i + 1] - kappas[i]) / (diff[i + 1] - diff[i])), kappas, ratio
    return None, kappas, ratio


def alpha_crossings(alphas: Sequence[float], **kw) -> Dict:
    """Crossing kappa per alpha, and the straight line kappa = slope / (2 alpha) + intercept through them with its R^2."""
    rows = []
    for a in alphas:
        k, _, _ = crossing_kappa(float(a), **kw)
        rows.append({"alpha": float(a), "inv_2alpha": 1.0 / (2 * a), "kappa": k})
    ok = [r for r in rows if r["kappa"] is not None]
    out = {"rows": rows}
    if len(ok) >= 2:
        x, y = np.array([r["inv_2alpha"] for r in ok]), np.array([r["kappa"] for r in ok])
        slope, icpt = np.polyfit(x, y, 1)
        tot = float(np.sum((y - y.mean()) ** 2))
        out["fit"] = {"slope": float(slope), "intercept": float(icpt),
                      "r_squared": 1.0 - float(np.sum((y - slope * x - icpt) ** 2)) / tot if tot > 0 else 1.0}
    return out


# ---- fixed against trajectory-driven g3 ---------------------------------------------------------------------------------
def _run_set(inp, sched, G1, G2, Dl, B, steps, dt, **kw):
    runs = {}
    for name, (g3, dyn) in sched.items():
        t, two_r, mom = solve_risk_ode(inp, DanaHparams(G1, G2, g3, Dl), B, steps, dt, momentum=True, dynamic_g3=dyn, **kw)
        risk = 0.5 * two_r
        with np.errstate(divide="ignore", invalid="ignore"):
            ratio = np.where(mom > 0, risk / np.maximum(mom, 1e-300), np.nan)
        runs[name] = {"t": t, "risk": risk, "momentum": mom, "risk_over_momentum": ratio,
                      "late_slope": loglog_slope(t, risk - inp.risk_infinity, steps ** 0.5, steps)}
    return runs


def dynamic_schedules(alpha: float = 0.7, beta: float = 0.5, v: int = 4000, d: int = 1000, h: float = 0.5, steps: float = 1e7,
                      dt: float = 1e-2) -> Dict:
    """Batch = d^h, momentum a raw sum (g1 = 1).  Runs: Dana-constant (g3 = 0.1 (B/d) lr), Dana-decay
    (g3 = 0.1 lr (1+t)^(-(1-h)/(2 alpha))), SGD, and the ratio rule on g3 = 0.5 lr."""
    B = int(d ** h)
    inp = ode_inputs(alpha, beta, v, d)
    lr = min(1.0, B / population_trace(alpha, v))
    sched = {"dana-constant": (const(0.1 * B / d * lr), None), "dana-decay": (powerlaw_schedule(0.1 * lr, 0.0, -(1.0 - h) / (2 * alpha), 1), None),
             "sgd": (const(0.0), None), "dynamic": (const(0.5 * lr), "ratio")}
    return {"args": dict(alpha=alpha, beta=beta, v=v, d=d, batch=B, steps=steps), "risk_infinity": inp.risk_infinity,
            "runs": _run_set(inp, sched, const(1.0), const(0.5 * lr), delta_schedule(alpha, beta), B, steps, dt)}


def danastar_schedules(alpha: float = 0.7, beta: float = 0.5, v: int = 4000, d: int = 1000, h: float = 0.0, steps: float = 1e7,
                       dt: float = 1e-2) -> Dict:
    """Every run divides g2 and g3 by sqrt(2 risk); momentum is a running mean (g1 = delta); lr = (0.1 / sqrt d) x the
    stable step.  Runs: g3 = 0.1 (B/d) lr (1+t), g3 = 0.1 lr (1+t)^(1 - (1-h)/(2 alpha)), SGD, and g3 = 0.5 lr / sqrt(2R)."""
    B = int(d ** h)
    inp = ode_inputs(alpha, beta, v, d)
    lr = 0.1 / math.sqrt(d) * min(1.0, B / population_trace(alpha, v))
    Dl = delta_schedule(alpha, beta)
    sched = {"dana-constant": (powerlaw_schedule(0.1 * B / d * lr, 0.0, 1.0, 1), None),
             "dana-decay": (powerlaw_schedule(0.1 * lr, 0.0, 1.0 - (1.0 - h) / (2 * alpha), 1), None),
             "sgd": (const(0.0), None), "dynamic": (const(0.5 * lr), "inv_sqrt_risk")}
    return {"args": dict(alpha=alpha, beta=beta, v=v, d=d, batch=B, steps=steps), "risk_infinity": inp.risk_infinity,
            "runs": _run_set(inp, sched, Dl, const(0.5 * lr), Dl, B, steps, dt, risk_renormalized=True, shifted_clock=True)}


# ---- command line --------------------------------------------------------------------------------------------------------
def _plain(o):
    if isinstance(o, dict):
        return {str(k): _plain(v) for k, v in o.items()}
    if isinstance(o, (list, tuple)):
        return [_plain(v) for v in o]
    if isinstance(o, np.ndarray):
        return [None if isinstance(x, float) and math.isnan(x) else x for x in o.tolist()]
    if isinstance(o, (np.floating, np.integer)):
        return o.item()
    return o


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="python -m adana_b200.theory.schedule_studies")
    sub = p.add_subparsers(dest="cmd", required=True)
    for name in ("compare", "kappa-sweep", "crossing", "dynamic"):
        s = sub.add_parser(name)
        s.add_argument("--alpha", type=float, default={"compare": 1.5, "kappa-sweep": 0.5, "dynamic": 0.7}.get(name, 0.5))
        s.add_argument("--beta", type=float, default=0.5 if name == "dynamic" else 0.3)
        s.add_argument("--d", type=int, default=300)
        s.add_argument("--v", type=int, default=None)
        s.add_argument("--steps", type=float, default=None)
        s.add_argument("--dt", type=float, default=1e-2)
        s.add_argument("--out", required=True)
        s.add_argument("--svg", default=None)
        if name == "crossing":
            s.add_argument("--alphas", type=float, nargs="+", default=[0.7, 0.825, 0.95, 1.075, 1.2])
        if name in ("kappa-sweep", "crossing"):
            s.add_argument("--num-kappa", type=int, default=20)
        if name == "dynamic":
            s.add_argument("--danastar", action="store_true")
            s.add_argument("--h", type=float, default=0.5)
    a = p.parse_args(argv)
    v = a.v or 4 * a.d
    if a.cmd == "compare":
        res = compare_optimizers(a.alpha, a.beta, a.d, v, steps=a.steps, dt=a.dt)
        series = {k: (r["t"], r["loss"]) for k, r in res["runs"].items()}
    elif a.cmd == "kappa-sweep":
        res = kappa_sweep(a.alpha, a.beta, v, a.d, steps=a.steps or 1e5, dt=a.dt, kappas=np.linspace(0, 1, a.num_kappa, endpoint=False))
        series = {f"kappa={r['kappa']:.2f}": (r["t"], r["risk"]) for r in res["runs"][::max(1, len(res["runs"]) // 8)]}
        series["dynamic g3"] = (res["dynamic"]["t"], res["dynamic"]["risk"])
    elif a.cmd == "crossing":
        res = alpha_crossings(a.alphas, beta=a.beta, v=v, d=a.d, steps=a.steps or 1e5, dt=a.dt,
                              kappas=np.linspace(-1.5, -0.2, a.num_kappa, endpoint=False))
        series = None
    else:
        res = (danastar_schedules if a.danastar else dynamic_schedules)(a.alpha, a.beta, v, a.d, a.h, a.steps or 1e6, a.dt)
        series = {k: (r["t"], r["risk"]) for k, r in res["runs"].items()}
    with open(a.out, "w") as f:
        json.dump(_plain(res), f)
    if a.svg:
        from ..figures import LineChart

        if series is None:
            rows = [r for r in res["rows"] if r["kappa"] is not None]
            ch = LineChart("self-consistent kappa against 1 / (2 alpha)", "1 / (2 alpha)", "crossing kappa")
            ch.add([r["inv_2alpha"] for r in rows], [r["kappa"] for r in rows], "crossing", markers=True)
            if "fit" in res:
                f = res["fit"]
                ch.add([r["inv_2alpha"] for r in rows], [f["slope"] * r["inv_2alpha"] + f["intercept"] for r in rows],
                       f"{f['slope']:.3f} / (2 alpha) + {f['intercept']:.3f}", dashed=True)
        else:
            ch = LineChart(f"{a.cmd}: risk against iterations", "iterations", "risk", logx=True, logy=True)
            for k, (t, y) in series.items():
                ch.add(t[t >= 1], y[t >= 1], k, dashed=k.startswith("dynamic"))
        ch.save(a.svg)
    print(f"wrote {a.out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
