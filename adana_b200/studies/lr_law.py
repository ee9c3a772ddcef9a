"""The learning-rate scaling law lr*(P) = a (b + P)^d: from the learning-rate sweeps of several model sizes to the
coefficients in `config/scaling_rules.yaml`, with bootstrap confidence intervals.

Pipeline (the reference's visualization/bighead_lr_scaling.py:347-446, 695-1102):
  1. per size, drop learning rates within 5 % of a better one (`dedupe_lrs`), keep the K best by final validation
     loss and weight them K, K-1, ..., 1 (`top_k_lrs`);
  2. fit log lr = log a + d log(b + P) over all kept points with weights w^2 * P (larger models count more);
  3. resample the sizes with replacement, refit, and read the percentile intervals of (a, b, d) and of the
     predicted lr at extrapolation sizes.

The fit here is exact for its objective: for a fixed b the weighted problem is linear in (log a, d), so b is found
by a scan in log b with a golden-section refinement, where the reference runs tens of thousands of Adagrad steps from
a fixed start.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np


def dedupe_lrs(rows: Sequence[Dict], tol: float = 0.05) -> List[Dict]:
    """Best-first pass: a row survives unless a better row's lr is within `tol` (relative to the larger of the two)."""
    kept: List[Dict] = []
    for r in sorted(rows, key=lambda r: r["val_loss"]):
        if all(abs(r["lr"] - k["lr"]) / max(r["lr"], k["lr"]) >= tol for k in kept):
            kept.append(r)
    return kept


def top_k_lrs(rows: Sequence[Dict], k: int = 5, omega: Optional[float] = None, omega_tol: float = 0.1,
              lr_tol: float = 0.05) -> Tuple[List[Dict], List[Dict]]:
    """-> (the K best rows with `weight` K..1, the other rows with `distance_from_optimal`)."""
    if omega is not None:
        rows = [r for r in rows if abs(r["omega"] - omega) < omega_tol]
    rows = dedupe_lrs(rows, lr_tol)
    if not rows:
        return [], []
    best = rows[0]["val_loss"]
    top = [dict(lr=r["lr"], val_loss=r["val_loss"], weight=k - i) for i, r in enumerate(rows[:k])]
    rest = [dict(lr=r["lr"], val_loss=r["val_loss"], distance_from_optimal=r["val_loss"] - best) for r in rows[k:]]
    return top, rest


def _solve_given_b(logb: float, P, y, w):
    X = np.stack([np.ones_like(P), np.log(math.exp(logb) + P)], axis=1)
    sw = np.sqrt(w)
    coef, *_ = np.linalg.lstsq(X * sw[:, None], y * sw, rcond=None)
    r = X @ coef - y
    return float(np.sum(w * r * r) / np.sum(w)), coef


def fit_weighted(params: Sequence[float], lrs: Sequence[float], weights: Optional[Sequence[float]] = None,
                 logb_range: Tuple[float, float] = (math.log(1e2), math.log(1e10))) -> Tuple[float, float, float, float]:
    """-> (a, b, d, weighted mean squared log-residual) of lr = a (b + P)^d with weights w^2 * P."""
    P = np.asarray(params, dtype=np.float64)
    y = np.log(np.asarray(lrs, dtype=np.float64))
    w = np.ones_like(P) if weights is None else np.asarray(weights, dtype=np.float64)
    w = w * w * P
    if len(np.unique(P)) < 2:
        raise ValueError("the law needs at least two different sizes")
    grid = np.linspace(logb_range[0], logb_range[1], 81)
    errs = [_solve_given_b(g, P, y, w)[0] for g in grid]
    k = int(np.argmin(errs))
    lo, hi = grid[max(k - 1, 0)], grid[min(k + 1, len(grid) - 1)]
    phi = (math.sqrt(5) - 1) / 2
    for _ in range(70):
        m1, m2 = hi - phi * (hi - lo), lo + phi * (hi - lo)
        if _solve_given_b(m1, P, y, w)[0] < _solve_given_b(m2, P, y, w)[0]:
            hi = m2
        else:
            lo = m1
    logb = 0.5 * (lo + hi)
    err, coef = _solve_given_b(logb, P, y, w)
    return float(math.exp(coef[0])), float(math.exp(logb)), float(coef[1]), err


def predict(P, a: float, b: float, d: float):
    return a * (b + np.asarray(P, dtype=np.float64)) ** d


def gather_points(per_size: Dict[int, Dict]) -> Tuple[List[float], List[float], List[float]]:
    """per_size: size -> {"non_emb_params": P, "top_k_data": [{lr, weight}, ...], optional "excluded": bool}."""
    P, lr, w = [], [], []
    for data in per_size.values():
        if data.get("excluded"):
            continue
        for item in data.get("top_k_data", []):
            P.append(data["non_emb_params"])
            lr.append(item["lr"])
            w.append(item["weight"])
    return P, lr, w


def bootstrap(per_size: Dict[int, Dict], n_boot: int = 1000, seed: int = 42):
    """Resample model sizes with replacement (a drawn size brings all of its top-K points); -> (a, b, d) sample arrays
    with NaN where a resample held a single size."""
    rng = np.random.default_rng(seed)
    sizes = [s for s, d in per_size.items() if not d.get("excluded") and d.get("top_k_data")]
    if len(sizes) < 2:
        raise ValueError(f"need at least 2 sizes with data for a bootstrap, got {len(sizes)}")
    out = np.full((3, n_boot), np.nan)
    for i in range(n_boot):
        draw = rng.choice(len(sizes), size=len(sizes), replace=True)
        sub = {j: per_size[sizes[k]] for j, k in enumerate(draw)}
        P, lr, w = gather_points(sub)
        try:
            out[:, i] = fit_weighted(P, lr, w)[:3]
        except (ValueError, np.linalg.LinAlgError):
            pass
    return out[0], out[1], out[2]


def _interval(x, level):
    lo, hi = 100 * (1 - level) / 2, 100 * (1 + level) / 2
    return {"mean": float(np.mean(x)), "std": float(np.std(x)), "median": float(np.median(x)),
            "ci_lower": float(np.percentile(x, lo)), "ci_upper": float(np.percentile(x, hi))}


def confidence_intervals(a_s, b_s, d_s, level: float = 0.95, extrapolate_to: Optional[Sequence[float]] = None) -> Dict:
    """Percentile intervals of the parameters and, per extrapolation size, of the predicted lr (keys as the
    reference's bootstrap JSON: parameters.{a,b,d}.{mean,std,median,ci_lower,ci_upper}, lr_predictions.<P>.lr_*)."""
    ok = ~(np.isnan(a_s) | np.isnan(b_s) | np.isnan(d_s))
    a, b, d = a_s[ok], b_s[ok], d_s[ok]
    res = {"confidence_level": level, "n_valid_samples": int(ok.sum()),
           "parameters": {"a": _interval(a, level), "b": _interval(b, level), "d": _interval(d, level)}}
    if extrapolate_to is not None:
        res["lr_predictions"] = {}
        for p in extrapolate_to:
            iv = _interval(a * (b + p) ** d, level)
            res["lr_predictions"][str(int(p))] = {"params": float(p), **{"lr_" + k: v for k, v in iv.items()}}
    return res


def confidence_band(P_range, a_s, b_s, d_s, level: float = 0.95):
    """-> (median, lower, upper) predicted lr along P_range."""
    ok = ~(np.isnan(a_s) | np.isnan(b_s) | np.isnan(d_s))
    a, b, d = a_s[ok], b_s[ok], d_s[ok]
    pred = a[None, :] * (b[None, :] + np.asarray(P_range, dtype=np.float64)[:, None]) ** d[None, :]
    lo, hi = 100 * (1 - level) / 2, 100 * (1 + level) / 2
    return np.median(pred, axis=1), np.percentile(pred, lo, axis=1), np.percentile(pred, hi, axis=1)


def study(table: Dict[int, List[Dict]], rule: str = "Enoki_Scaled", k: int = 5, omega: Optional[float] = None,
          n_boot: int = 0, exclude: Sequence[int] = (), extrapolate_sizes: Sequence[int] = (), seed: int = 42) -> Dict:
    """The whole pipeline from a `runs.lr_sweep_table`: per-size top-K, the fitted law, optional bootstrap."""
    from .sizes import model_size

    per_size = {}
    for size, rows in sorted(table.items()):
        top, rest = top_k_lrs(rows, k, omega)
        if top:
            per_size[size] = {"non_emb_params": model_size(size, rule).non_emb, "top_k_data": top, "others": rest,
                              "excluded": size in exclude}
    a, b, d, err = fit_weighted(*gather_points(per_size))
    out = {"metadata": {"scaling_rule": rule, "target_omega": omega, "top_k": k},
           "fit": {"a": a, "b": b, "d": d, "weighted_mse_log": err}, "sizes": per_size}
    if n_boot:
        a_s, b_s, d_s = bootstrap(per_size, n_boot, seed)
        out["bootstrap"] = confidence_intervals(a_s, b_s, d_s, extrapolate_to=[model_size(s, rule).non_emb
                                                                               for s in extrapolate_sizes])
    return out
