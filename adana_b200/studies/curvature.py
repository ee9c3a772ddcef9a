"""How sharp the loss is around the best learning rate, per model size, and what a mis-set learning rate costs.

For every size the sweep's (lr, final validation loss) points are fitted with a parabola in log lr,
    loss(lr) = L* + kappa (log lr - log lr*)^2,
kappa being the curvature.  Across sizes the curvatures are summarised by their mean (and, for comparison, by a power
law kappa0 P^alpha, which the reference keeps but calls unreliable); an lr that is off by a fraction eps then costs
    delta loss = kappa (log(1 + eps))^2.

Reference: visualization/lr_curvature_analysis.py:275-400; the JSON written by `study` has the keys its consumer
(compute_saved_sensitivity.py) reads: `curvature_scaling_law.{kappa_0, alpha}`, `loss_sensitivity.extrapolation_sizes`.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np


def fit_parabola(lrs: Sequence[float], losses: Sequence[float]) -> Tuple[float, float, float]:
    """-> (L*, lr*, kappa); NaNs when no convex fit exists.  If the fit over all points opens downwards, the three
    (at the ends of the sweep: up to five) points around the best one are tried."""
    x, y = np.log(np.asarray(lrs, dtype=np.float64)), np.asarray(losses, dtype=np.float64)
    a, b, c = np.polyfit(x, y, 2)
    if a <= 0:
        i, n = int(np.argmin(y)), len(y)
        lo, hi = max(0, i - 1), min(n, i + 2)
        if hi - lo < 3:
            lo, hi = max(0, i - 2), min(n, i + 3)
        if hi - lo >= 3:
            a, b, c = np.polyfit(x[lo:hi], y[lo:hi], 2)
    if a <= 0:
        return math.nan, math.nan, math.nan
    return float(c - b * b / (4 * a)), float(math.exp(-b / (2 * a))), float(a)


def mean_curvature(curvatures: Sequence[float]) -> Tuple[float, float]:
    k = np.asarray(curvatures, dtype=np.float64)
    k = k[~np.isnan(k)]
    return (float(k.mean()), float(k.std())) if len(k) else (math.nan, math.nan)


def curvature_power_law(params: Sequence[float], curvatures: Sequence[float]) -> Tuple[float, float]:
    """-> (kappa0, alpha) of kappa = kappa0 P^alpha by a straight line in log-log; NaNs with fewer than two sizes."""
    P, k = np.asarray(params, dtype=np.float64), np.asarray(curvatures, dtype=np.float64)
    ok = ~np.isnan(k)
    if ok.sum() < 2:
        return math.nan, math.nan
    alpha, logk0 = np.polyfit(np.log(P[ok]), np.log(k[ok]), 1)
    return float(math.exp(logk0)), float(alpha)


def loss_increase(lr_error: float, kappa: float) -> float:
    """Loss paid for a learning rate that is off by the fraction `lr_error`."""
    return float(kappa * math.log(1.0 + lr_error) ** 2)


def loss_increase_at(params: float, lr_error: float, kappa0: float, alpha: float) -> float:
    return loss_increase(lr_error, kappa0 * params ** alpha)


def study(table: Dict[int, List[Dict]], rule: str = "Enoki_Scaled", lr_errors: Sequence[float] = (0.1, 0.2, 0.5),
          extrapolation_sizes: Optional[Sequence[int]] = None, min_points: int = 3) -> Dict:
    """From a `runs.lr_sweep_table` (size -> rows with lr and val_loss) to the curvature report."""
    from .lr_law import dedupe_lrs
    from .sizes import model_size

    per_size, P, K = {}, [], []
    for size, rows in sorted(table.items()):
        rows = sorted(dedupe_lrs(rows), key=lambda r: r["lr"])
        if len(rows) < min_points:
            continue
        L, lr_star, kappa = fit_parabola([r["lr"] for r in rows], [r["val_loss"] for r in rows])
        n = model_size(size, rule).non_emb
        per_size[str(size)] = {"non_emb_params": n, "n_points": len(rows), "L_star": L, "lr_star": lr_star, "kappa": kappa}
        P.append(n)
        K.append(kappa)
    mean, std = mean_curvature(K)
    k0, alpha = curvature_power_law(P, K)
    sizes = list(extrapolation_sizes or sorted(table))
    sens = {str(s): {f"{e:g}": {"mean_kappa": loss_increase(e, mean),
                               "power_law": loss_increase_at(model_size(s, rule).non_emb, e, k0, alpha)}
                     for e in lr_errors} for s in sizes}
    return {"metadata": {"scaling_rule": rule}, "per_size": per_size,
            "average_curvature": {"mean": mean, "std": std},
            "curvature_scaling_law": {"kappa_0": k0, "alpha": alpha},
            "loss_sensitivity": {"extrapolation_sizes": sizes, "lr_errors": list(lr_errors), "delta_loss": sens}}
