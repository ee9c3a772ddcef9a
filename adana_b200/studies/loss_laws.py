"""Loss as a function of training compute: the three laws the scaling comparison fits, alone or jointly over several
optimizers with one shared floor, and the compute multiplier one optimizer has over another.

    single      L = a + b C^-c                 (a free, or forced to 0)
    broken      L = a + b C^-c + e C^-f        (two regimes)
    joint       the same forms fitted to several curves at once: a is shared, the rest is per curve; residuals are
                taken in log L, optionally weighted by compute

Reference: visualization/compute_formula_comparison.py:71-219 (single and broken fits, loss-space residuals),
compute_formula_residuals.py:76-209 (broken with a given shared floor), compare_scaling_rules_ep.py:681-1156 (joint
fits with a = lower + sigmoid(.) * (0.99 min loss - lower)) and :1905-2045 (compute multiplier, piecewise and from the
fitted curves).  The reference minimises with 30-50 thousand Adagrad steps from fixed starts; here the fits are
non-linear least squares (trust-region, analytic structure where there is some) from several starts, which reaches
the same minima in milliseconds and does not depend on a step count.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Sequence

import numpy as np
from scipy.optimize import brentq, least_squares, nnls


def single(C, a, b, c):
    return a + b * np.power(C, -c)


def broken(C, a, b, c, e, f):
    return a + b * np.power(C, -c) + e * np.power(C, -f)


def r_squared(y, pred) -> float:
    y, pred = np.asarray(y, dtype=np.float64), np.asarray(pred, dtype=np.float64)
    tot = float(np.sum((y - y.mean()) ** 2))
    return 1.0 - float(np.sum((y - pred) ** 2)) / tot if tot > 0 else 0.0


def _report(C, L, pred, **params) -> Dict:
    return {**{k: float(v) for k, v in params.items()}, "r_squared": r_squared(L, pred),
            "predictions": np.asarray(pred), "residuals": np.asarray(L) - np.asarray(pred)}


def fit_single(C: Sequence[float], L: Sequence[float], force_a_zero: bool = False) -> Dict:
    """Least squares in loss space.  For a fixed exponent the model is linear in (a, b) with b >= 0, so the exponent
    is scanned and the linear part solved exactly (non-negative least squares), then all three are polished."""
    C, L = np.asarray(C, dtype=np.float64), np.asarray(L, dtype=np.float64)

    def linear_part(c):
        cols = [np.power(C, -c)] if force_a_zero else [np.ones_like(C), np.power(C, -c)]
        coef, res = nnls(np.stack(cols, axis=1), L)
        return res, coef

    grid = np.linspace(0.005, 1.5, 300)
    c0 = float(grid[int(np.argmin([linear_part(c)[0] for c in grid]))])
    coef = linear_part(c0)[1]
    a0, b0 = (0.0, coef[0]) if force_a_zero else (coef[0], coef[1])
    if force_a_zero:
        sol = least_squares(lambda p: math.exp(p[0]) * np.power(C, -p[1]) - L, [math.log(max(b0, 1e-12)), c0])
        a, b, c = 0.0, math.exp(sol.x[0]), sol.x[1]
    else:
        sol = least_squares(lambda p: p[0] + math.exp(p[1]) * np.power(C, -p[2]) - L, [a0, math.log(max(b0, 1e-12)), c0])
        a, b, c = sol.x[0], math.exp(sol.x[1]), sol.x[2]
    return _report(C, L, single(C, a, b, c), a=a, b=b, c=c)


_BROKEN_STARTS = [(0.5, 0.05, 0.1, 0.2), (0.4, 0.2, 2.5, 0.03), (1.0, 0.1, 1.0, 0.5), (0.1, 0.3, 3.0, 0.05)]


def fit_broken(C: Sequence[float], L: Sequence[float], a: Optional[float] = None) -> Dict:
    """L = a + b C^-c + e C^-f in loss space; `a` free, or given (a floor shared with other curves)."""
    C, L = np.asarray(C, dtype=np.float64), np.asarray(L, dtype=np.float64)
    best = None
    for b0, c0, e0, f0 in _BROKEN_STARTS:
        if a is None:
            fun = lambda p: broken(C, p[0], math.exp(p[1]), p[2], math.exp(p[3]), p[4]) - L
            x0 = [0.1, math.log(b0), c0, math.log(e0), f0]
        else:
            fun = lambda p: broken(C, a, math.exp(p[0]), p[1], math.exp(p[2]), p[3]) - L
            x0 = [math.log(b0), c0, math.log(e0), f0]
        sol = least_squares(fun, x0, max_nfev=4000)
        if best is None or sol.cost < best.cost:
            best = sol
    p = best.x if a is not None else best.x[1:]
    a_fit = a if a is not None else best.x[0]
    b, c, e, f = math.exp(p[0]), p[1], math.exp(p[2]), p[3]
    return _report(C, L, broken(C, a_fit, b, c, e, f), a=a_fit, b=b, c=c, e=e, f=f)


def _sigmoid(x):
    return 1.0 / (1.0 + math.exp(-x))


def fit_joint(curves: Sequence[Dict], form: str = "broken", a_lower: float = 0.0, a_upper: Optional[float] = None,
              compute_weight: bool = False) -> Dict:
    """Several curves, one floor.  `curves`: dicts with `name`, `compute`, `loss`.  The floor is kept between
    `a_lower` and `a_upper` (default: 99 % of the smallest loss seen) through a sigmoid; residuals are differences of
    log loss, weighted by compute when `compute_weight`.  -> {"a": floor, "curves": {name: {b, c[, e, f], r_squared}}}."""
    if form not in ("single", "broken"):
        raise ValueError("form is 'single' or 'broken'")
    data = [(d["name"], np.asarray(d["compute"], dtype=np.float64), np.asarray(d["loss"], dtype=np.float64)) for d in curves]
    top = 0.99 * min(float(L.min()) for _, _, L in data) if a_upper is None else a_upper
    k = 2 if form == "single" else 4
    total_w = sum(float(C.sum()) if compute_weight else len(C) for _, C, _ in data)

    def unpack(p, i):
        q = p[1 + k * i: 1 + k * (i + 1)]
        return (math.exp(q[0]), q[1]) if form == "single" else (math.exp(q[0]), q[1], math.exp(q[2]), q[3])

    def floor(p):
        return a_lower + _sigmoid(p[0]) * (top - a_lower)

    def resid(p):
        a, out = floor(p), []
        for i, (_, C, L) in enumerate(data):
            pred = single(C, a, *unpack(p, i)) if form == "single" else broken(C, a, *unpack(p, i))
            w = np.sqrt((C if compute_weight else np.ones_like(C)) / total_w)
            out.append(w * (np.log(np.maximum(pred, 1e-10)) - np.log(L)))
        return np.concatenate(out)

    starts = [(0.5, 0.1)] if form == "single" else [(0.4, 0.2, 2.5, 0.03), (0.5, 0.05, 0.1, 0.2)]
    best = None
    for s in starts:
        for a_raw in (-3.1, 0.0):
            per = [math.log(s[0]), s[1]] if form == "single" else [math.log(s[0]), s[1], math.log(s[2]), s[3]]
            sol = least_squares(resid, [a_raw] + per * len(data), max_nfev=6000)
            if best is None or sol.cost < best.cost:
                best = sol
    a = floor(best.x)
    out = {"a": float(a), "form": form, "curves": {}}
    for i, (name, C, L) in enumerate(data):
        q = unpack(best.x, i)
        pred = single(C, a, *q) if form == "single" else broken(C, a, *q)
        keys = ("b", "c") if form == "single" else ("b", "c", "e", "f")
        out["curves"][name] = {**dict(zip(keys, map(float, q))), "r_squared": r_squared(L, pred)}
    return out


# ---- compute multiplier ----------------------------------------------------------------------------------------------
def baseline_compute_for_loss(loss: float, base_C: Sequence[float], base_L: Sequence[float]) -> float:
    """Compute the baseline needs for `loss`, reading its measured points as a piecewise-linear curve in log-log and
    extending the first / last segment beyond them."""
    C, L = np.asarray(base_C, dtype=np.float64), np.asarray(base_L, dtype=np.float64)
    order = np.argsort(C)
    lc, ll, t = np.log(C[order]), np.log(L[order]), math.log(loss)
    if len(lc) < 2:
        return math.nan
    if L.min() <= loss <= L.max():
        return float(math.exp(np.interp(t, ll[::-1], lc[::-1]) if ll[0] > ll[-1] else np.interp(t, ll, lc)))
    i, j = (-2, -1) if loss < L.min() else (0, 1)
    slope = (lc[j] - lc[i]) / (ll[j] - ll[i])
    anchor = j if loss < L.min() else i
    return float(math.exp(lc[anchor] + slope * (t - ll[anchor])))


def multiplier_piecewise(opt_C, opt_L, base_C, base_L):
    """For every measured point of an optimizer: baseline compute at equal loss / the optimizer's compute.
    -> (compute, multiplier) arrays sorted by compute; > 1 means the optimizer is cheaper."""
    C = np.asarray(opt_C, dtype=np.float64)
    g = np.array([baseline_compute_for_loss(l, base_C, base_L) for l in opt_L]) / C
    ok = np.isfinite(g)
    order = np.argsort(C[ok])
    return C[ok][order], g[ok][order]


def multiplier_from_fits(C_range, a: float, opt: Dict, base: Dict):
    """The same ratio from two fitted broken laws with the shared floor `a`: for each C, the optimizer's fitted loss
    is matched on the baseline's curve by root finding in log compute."""
    xs, out = [], []
    for C in np.asarray(C_range, dtype=np.float64):
        L = broken(C, a, opt["b"], opt["c"], opt["e"], opt["f"])
        if L <= a:
            continue
        g = lambda lc: broken(math.exp(lc), a, base["b"], base["c"], base["e"], base["f"]) - L
        try:
            xs.append(C)
            out.append(math.exp(brentq(g, -10, 30)) / C)
        except ValueError:
            xs.pop()
    return np.array(xs), np.array(out)
