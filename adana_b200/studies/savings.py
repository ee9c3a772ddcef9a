"""Compute saved against a baseline optimizer, and how much of that claim survives the uncertainty of the predicted
learning rate.

Measured savings (the reference's visualization/compute_saved.py:458-515, 627-690): per model size, take the
baseline's final loss, find the first point of the candidate's validation curve (against compute in PFLOP-hours) at or
below it, and count the compute the candidate still had to go; over sizes the savings follow saved = b X^c, fitted as
a straight line of log(saved + 1) against log X inside a compute window.

Sensitivity (compute_saved_sensitivity.py:85-330): with the loss law L = a + b C^-c inverted to C(L), a loss difference
becomes a compute ratio; the bootstrap interval of the predicted lr (studies.lr_law) becomes an lr error, the
curvature (studies.curvature) turns that into a loss spread, and the spread into an interval of the saved fraction.
"""
from __future__ import annotations

import math
from statistics import NormalDist
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np


# ---- measured ---------------------------------------------------------------------------------------------------------
def first_crossing(history: Sequence[Tuple[float, float]], target_loss: float) -> Optional[float]:
    """Compute at the first (compute, loss) record whose loss is <= target_loss."""
    for c, l in history:
        if l <= target_loss:
            return float(c)
    return None


def saved_per_size(baselines: Dict[int, Dict], candidates: Dict[int, List[Dict]]) -> List[Dict]:
    """baselines: size -> {final_loss, final_compute, model_compute, non_emb}; candidates: size -> runs, each
    {history: [(compute, loss)...], final_compute, run_name}.  Of the candidate runs that reach the baseline's final
    loss the one that reaches it earliest counts."""
    out = []
    for size, base in baselines.items():
        best = None
        for run in candidates.get(size, []):
            x = first_crossing(run["history"], base["final_loss"])
            if x is not None and (best is None or x < best[0]):
                best = (x, run["final_compute"], run.get("run_name"))
        if best:
            out.append({"size": size, "compute_saved": best[1] - best[0], "crossing_compute": best[0],
                        "final_compute": best[1], "adamw_final_loss": base["final_loss"],
                        "model_compute": base.get("model_compute"), "non_emb": base.get("non_emb"), "run_name": best[2]})
    return out


def fit_savings_lines(datasets: Sequence[Dict], compute_range: Tuple[float, float] = (1.0, 30.0)) -> Dict:
    """saved = b X^c per dataset ({name, x, y}) from the points with compute_range[0] <= x <= compute_range[1]."""
    res = {"curves": {}}
    for d in datasets:
        x, y = np.asarray(d["x"], dtype=np.float64), np.asarray(d["y"], dtype=np.float64)
        m = (x >= compute_range[0]) & (x <= compute_range[1])
        if m.sum() < 2:
            continue
        c, logb = np.polyfit(np.log(x[m]), np.log(y[m] + 1), 1)
        pred = math.exp(logb) * x[m] ** c
        tot = float(np.sum((y[m] - y[m].mean()) ** 2))
        res["curves"][d["name"]] = {"b": float(math.exp(logb)), "c": float(c), "n_points": int(m.sum()),
                                    "r_squared": 1 - float(np.sum((y[m] - pred) ** 2)) / tot if tot > 0 else 0.0,
                                    "compute_range": tuple(compute_range)}
    return res


# ---- from the loss law ------------------------------------------------------------------------------------------------
def loss_at(compute: float, a: float, b: float, c: float) -> float:
    return a + b * compute ** (-c)


def compute_for(loss: float, a: float, b: float, c: float) -> float:
    """Inverse of the loss law; infinite at or below the floor."""
    return math.inf if loss <= a else ((loss - a) / b) ** (-1.0 / c)


def saved(baseline_loss: float, opt_loss: float, a: float, b: float, c: float) -> float:
    return compute_for(baseline_loss, a, b, c) - compute_for(opt_loss, a, b, c)


def saved_fraction(baseline_loss: float, opt_loss: float, a: float, b: float, c: float) -> float:
    """(C(baseline loss) - C(candidate loss)) / C(baseline loss) on one law.  With the candidate's loss below the
    baseline's this is negative (the law needs more compute for the lower loss): its size is the extra compute the
    baseline would have to spend to catch up, in units of what it spent."""
    cb = compute_for(baseline_loss, a, b, c)
    return (cb - compute_for(opt_loss, a, b, c)) / cb


def lr_error_from_interval(lr_mean: float, lo: float, hi: float) -> float:
    """Mean of the two relative half-widths of the interval."""
    return (abs(lr_mean - lo) / lr_mean + abs(hi - lr_mean) / lr_mean) / 2


def saved_fraction_interval(baseline_loss: float, opt_loss: float, opt_loss_std: float, a: float, b: float, c: float,
                            level: float = 0.95) -> Dict[str, float]:
    """Gaussian spread of the candidate's loss pushed through the law: the low end of the loss interval is the
    optimistic end of the savings."""
    z = NormalDist().inv_cdf((1 + level) / 2)
    lo, hi = opt_loss - z * opt_loss_std, opt_loss + z * opt_loss_std
    return {"mean": saved_fraction(baseline_loss, opt_loss, a, b, c),
            "ci_lower": saved_fraction(baseline_loss, hi, a, b, c),
            "ci_upper": saved_fraction(baseline_loss, lo, a, b, c),
            "loss_mean": opt_loss, "loss_ci_lower": lo, "loss_ci_upper": hi}


def loss_spread_from_lr(bootstrap: Dict, curvature: Dict, target_params: float):
    """-> (loss spread taken as one standard deviation, lr error) at `target_params`, from a bootstrap report
    (`lr_predictions` keyed by parameter count; the nearest key is used) and a curvature report."""
    from .curvature import loss_increase

    preds = bootstrap.get("lr_predictions", {})
    if not preds:
        return None, None
    key = min(preds, key=lambda k: abs(int(k) - target_params))
    p = preds[key]
    err = lr_error_from_interval(p["lr_mean"], p["lr_ci_lower"], p["lr_ci_upper"])
    law = curvature["curvature_scaling_law"]
    return loss_increase(err, law["kappa_0"] * target_params ** law["alpha"]), err


def sensitivity(bootstraps: Dict[str, Dict], curvature: Dict, losses: Dict[str, float], baseline: str,
                target_params: float, a: float, b: float, c: float, level: float = 0.95) -> Dict:
    """Per optimizer: lr error, loss spread, and the saved fraction against `baseline` with its interval.
    `losses` maps optimizer -> loss at the target scale (measured or read off its loss law)."""
    out = {"confidence_level": level, "baseline": baseline, "target_params": target_params, "analysis": []}
    for name, boot in bootstraps.items():
        std, err = loss_spread_from_lr(boot, curvature, target_params)
        row = {"optimizer": name, "lr_error": err, "loss_std": std}
        if name != baseline and std is not None:
            row["compute_saved"] = saved_fraction_interval(losses[baseline], losses[name], std, a, b, c, level)
        out["analysis"].append(row)
    return out
