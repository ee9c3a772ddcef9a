"""How the best `gamma_3_factor` (the multiplier of the long-momentum term) moves with the length of training.

Runs of one model size are grouped by iteration count; inside a group of at least three runs they are ranked by final
validation loss, the K best are kept with weights n - rank (n runs in the group), and a curve gamma3(T) is fitted to
the kept points of all sizes: a power law a T^b (weighted line in log-log), a line, an exponential, or the forms
delta T^kappa and T^(+-kappa) that tie the factor to the optimizer's kappa.

Reference: visualization/gamma3_factor_scaling.py:354-415 (window in multiples of the Chinchilla iteration count),
:418-615 (fit forms), :660-720 (ranking and weights).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .sizes import model_size


def within_chinchilla_window(rows: Sequence[Dict], rule: str, fac_min: float = 0.0, fac_max: float = math.inf) -> List[Dict]:
    """Rows ({size, iterations, ...}) whose iteration count lies in [fac_min, fac_max] x the Chinchilla count."""
    out = []
    for r in rows:
        f = r["iterations"] / model_size(r["size"], rule).chinchilla_iterations()
        if fac_min <= f <= fac_max:
            out.append(r)
    return out


def ranked_points(rows: Sequence[Dict], top_k: int = 5, min_runs: int = 3) -> List[Dict]:
    """Rows {size, iterations, gamma_3_factor, val_loss} -> the kept rows with `rank` and `weight`."""
    groups: Dict[Tuple[int, int], List[Dict]] = {}
    for r in rows:
        groups.setdefault((r["size"], r["iterations"]), []).append(r)
    kept = []
    for (_, _), g in sorted(groups.items()):
        if len(g) < min_runs:
            continue
        for rank, r in enumerate(sorted(g, key=lambda r: r["val_loss"])[:top_k]):
            kept.append({**r, "rank": rank, "weight": len(g) - rank})
    return kept


def _valid(T, g, w):
    T, g = np.asarray(T, dtype=np.float64), np.asarray(g, dtype=np.float64)
    w = np.ones_like(T) if w is None else np.asarray(w, dtype=np.float64)
    return T, g, w


def fit(T, g, kind: str = "power", weights=None) -> Optional[Tuple[float, float]]:
    """power: g = a T^b -> (a, b); linear: g = a T + b -> (a, b); exponential: g = a exp(b T) -> (a, b).  Weights
    multiply the residuals (as in a weighted polynomial fit); None with fewer than two usable points."""
    T, g, w = _valid(T, g, weights)
    if kind == "power":
        m = (T > 0) & (g > 0) & (w > 0) & np.isfinite(T) & np.isfinite(g)
        if m.sum() < 2:
            return None
        b, loga = np.polyfit(np.log(T[m]), np.log(g[m]), 1, w=w[m])
        return float(math.exp(loga)), float(b)
    if kind == "linear":
        m = np.isfinite(T) & np.isfinite(g) & (w > 0)
        if m.sum() < 2:
            return None
        a, b = np.polyfit(T[m], g[m], 1, w=w[m])
        return float(a), float(b)
    if kind == "exponential":
        m = (g > 0) & np.isfinite(T) & np.isfinite(g) & (w > 0)
        if m.sum() < 2:
            return None
        b, loga = np.polyfit(T[m], np.log(g[m]), 1, w=w[m])
        return float(math.exp(loga)), float(b)
    raise ValueError(f"unknown fit kind {kind!r} (power, linear, exponential)")


def evaluate(T, params: Tuple[float, float], kind: str = "power"):
    T = np.asarray(T, dtype=np.float64)
    a, b = params
    return a * T ** b if kind == "power" else a * T + b if kind == "linear" else a * np.exp(b * T)


def fit_delta_kappa(T, g, weights=None):
    """g = delta T^kappa -> ((delta, kappa), per-point kappa_i = log g_i / log T_i)."""
    T, g, w = _valid(T, g, weights)
    m = (T > 0) & (g > 0) & (w > 0) & np.isfinite(T) & np.isfinite(g)
    if m.sum() < 2:
        return None, None
    kappa, logd = np.polyfit(np.log(T[m]), np.log(g[m]), 1, w=w[m])
    return (float(math.exp(logd)), float(kappa)), np.log(g[m]) / np.log(T[m])


def fit_kappa_only(T, g, weights=None, negative: bool = False) -> Optional[float]:
    """g = T^kappa (or T^-kappa with `negative`): weighted line through the origin in log-log."""
    T, g, w = _valid(T, g, weights)
    m = (T > 0) & (g > 0) & (w > 0) & np.isfinite(T) & np.isfinite(g)
    if m.sum() < 2:
        return None
    x, y = np.log(T[m]), np.log(g[m])
    den = float(np.sum(w[m] * x * x))
    if den == 0:
        return None
    k = float(np.sum(w[m] * x * y)) / den
    return -k if negative else k


def study(rows: Sequence[Dict], rule: str = "Enoki_Scaled", top_k: int = 5, kind: str = "power",
          fac_min: float = 0.0, fac_max: float = math.inf) -> Dict:
    rows = within_chinchilla_window(rows, rule, fac_min, fac_max)
    pts = ranked_points(rows, top_k)
    T = [p["iterations"] for p in pts]
    g = [p["gamma_3_factor"] for p in pts]
    w = [p["weight"] for p in pts]
    dk, per_point = fit_delta_kappa(T, g, w)
    return {"points": pts, "kind": kind, "params": fit(T, g, kind, w), "delta_kappa": dk,
            "kappa_only": fit_kappa_only(T, g, w), "kappa_only_negative": fit_kappa_only(T, g, w, negative=True),
            "per_point_kappa": None if per_point is None else per_point.tolist()}
