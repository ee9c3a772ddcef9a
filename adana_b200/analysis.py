"""Numbers the paper-figure scripts derive from training logs, as plain functions over `metrics.jsonl`
records (or any lists): compute in PFLOP-hours, GPU-hours, compute saved at equal loss, and the optimal-LR
power-law fit that produces the coefficients of `config/scaling_rules.yaml`.

Counterparts in the reference's `visualization/` tree (which reads the W&B API and draws matplotlib figures):
compute = 6 * non_emb * tokens, PFH = / 3600e15 (compute_saved.py:232-233, 325-328); GPU-hours = mean iter_dt *
iters * world / 3600 (compute_gpu_hours.py:383-394); the LR law lr = a * (b + P)^d with a bootstrap over sizes
(bighead_lr_scaling.py).  `adana_b200.figures` draws the figures from these numbers; the metric names they read
(`iter`, `tokens`, `train/loss`, `val/loss`, `final-val/loss`, `iter_dt`, `lr`) are the ones the trainer logs.

    python -m adana_b200.analysis summary <exp_dir> [--non_emb N] [--world W]
"""
from __future__ import annotations

import argparse
import json
import math
from pathlib import Path
from typing import Dict, Iterable, Optional, Sequence, Tuple

import numpy as np

from .logging.metrics import read_metrics, series

PFH = 3600e15


def compute_pfh(non_emb_params: float, tokens: float) -> float:
    """Training compute in PetaFLOP-hours: 6 * P_non_emb * tokens / 3600e15."""
    return 6.0 * non_emb_params * tokens / PFH


def chinchilla_compute_pfh(non_emb_params: float, total_params: float, tokens_per_param: float = 20.0) -> float:
    """Compute of a Chinchilla-budget run (tokens = 20 * total parameters)."""
    return compute_pfh(non_emb_params, tokens_per_param * total_params)


def gpu_hours(iter_dts: Iterable[float], iterations: int, world_size: int) -> float:
    dts = [d for d in iter_dts if d is not None and math.isfinite(d)]
    return (sum(dts) / len(dts)) * iterations * world_size / 3600.0 if dts else float("nan")


def loss_vs_compute(rows: Sequence[Dict], non_emb_params: float, key: str = "val/loss"):
    """-> (compute in PFH, loss) arrays from metric records that carry `tokens` and `key`."""
    xs, ys = series(rows, key, x="tokens")
    c = np.array([compute_pfh(non_emb_params, t) for t in xs])
    return c, np.array(ys, dtype=np.float64)


def compute_to_reach(compute: np.ndarray, loss: np.ndarray, target: float) -> float:
    """Smallest compute at which the (running-best) loss curve reaches `target`, interpolating linearly in
    log-compute between the two bracketing points; NaN if it never does."""
    best = np.minimum.accumulate(loss)
    hit = np.nonzero(best <= target)[0]
    if len(hit) == 0:
        return float("nan")
    i = int(hit[0])
    if i == 0 or compute[i - 1] <= 0:
        return float(compute[i])
    l0, l1 = best[i - 1], best[i]
    w = 0.0 if l0 == l1 else (l0 - target) / (l0 - l1)
    return float(math.exp(math.log(compute[i - 1]) + w * (math.log(compute[i]) - math.log(compute[i - 1]))))


def compute_saved(baseline: Tuple[np.ndarray, np.ndarray], candidate: Tuple[np.ndarray, np.ndarray]) -> float:
    """Fraction of the baseline's final compute that the candidate does NOT need to reach the baseline's final
    loss (positive = candidate is cheaper)."""
    bc, bl = baseline
    target = float(np.min(bl))
    need = compute_to_reach(candidate[0], candidate[1], target)
    return float("nan") if math.isnan(need) else 1.0 - need / float(bc[-1])


def fit_lr_power_law(non_emb: Sequence[float], best_lr: Sequence[float], b_grid: Optional[Sequence[float]] = None):
    """Least squares in log space of lr = a * (b + P)^d.  For fixed b the problem is linear in (log a, d); b is
    scanned on a log grid and refined by golden-section search.  Returns (a, b, d, rms log-residual)."""
    P = np.asarray(non_emb, dtype=np.float64)
    y = np.log(np.asarray(best_lr, dtype=np.float64))

    def solve(b):
        X = np.stack([np.ones_like(P), np.log(b + P)], axis=1)
        coef, *_ = np.linalg.lstsq(X, y, rcond=None)
        r = X @ coef - y
        return float(np.sqrt(np.mean(r * r))), coef

    grid = np.geomspace(1e2, 1e8, 61) if b_grid is None else np.asarray(b_grid, dtype=np.float64)
    errs = [solve(b)[0] for b in grid]
    k = int(np.argmin(errs))
    lo, hi = grid[max(k - 1, 0)], grid[min(k + 1, len(grid) - 1)]
    phi = (math.sqrt(5) - 1) / 2
    for _ in range(60):
        m1, m2 = hi - phi * (hi - lo), lo + phi * (hi - lo)
        if solve(m1)[0] < solve(m2)[0]:
            hi = m2
        else:
            lo = m1
    b = 0.5 * (lo + hi)
    err, coef = solve(b)
    return float(math.exp(coef[0])), float(b), float(coef[1]), err


def bootstrap_lr_law(non_emb, best_lr, n_boot: int = 200, seed: int = 0):
    """Resample sizes with replacement; returns the point estimate and the (a, b, d) samples."""
    rng = np.random.default_rng(seed)
    P, lr = np.asarray(non_emb, dtype=np.float64), np.asarray(best_lr, dtype=np.float64)
    point = fit_lr_power_law(P, lr)
    samples = []
    for _ in range(n_boot):
        idx = rng.integers(0, len(P), len(P))
        if len(set(idx.tolist())) < 3:
            continue
        samples.append(fit_lr_power_law(P[idx], lr[idx])[:3])
    return point, np.array(samples)


def summarize_run(exp_dir, non_emb: Optional[float] = None, world: int = 1) -> Dict:
    rows = read_metrics(exp_dir)
    out: Dict = {"records": len(rows)}
    for key in ("train/loss", "val/loss", "final-val/loss"):
        _, ys = series(rows, key)
        if ys:
            out[key] = {"last": ys[-1], "best": min(ys)}
    _, dts = series(rows, "iter_dt")
    its, _ = series(rows, "train/loss")
    if dts and its:
        out["gpu_hours"] = gpu_hours(dts, max(its), world)
    toks, _ = series(rows, "train/loss", x="tokens")
    if non_emb and toks:
        out["compute_pfh"] = compute_pfh(non_emb, max(toks))
    return out


def main(argv=None) -> int:
    p = argparse.ArgumentParser()
    sub = p.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("summary")
    s.add_argument("exp_dir")
    s.add_argument("--non_emb", type=float, default=None)
    s.add_argument("--world", type=int, default=1)
    a = p.parse_args(argv)
    print(json.dumps(summarize_run(Path(a.exp_dir), a.non_emb, a.world), indent=1))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
