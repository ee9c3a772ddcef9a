"""Shared-gradient optimizer comparisons and sweeps on the power-law random-features problem.

The reference's experiment scripts (jax/moe_m_sweeps*.py, lr_m_sweeps.py, taustats_generate.py, kappa_sweep_plot.py)
train several optimizers side by side on the SAME stream of batches, sweep one hyper-parameter, and record the
order statistics of Dana-Star's tau estimate.  These are the numerical parts of those scripts as functions; the
figures are not reproduced.

* `compare_rules`        every rule gets its own weights but sees the same batches (same seed), so differences
                         between curves are due to the update rule alone.
* `sweep`                one rule factory over a list of values of one hyper-parameter (kappa, learning rate, ...).
* `final_risk_exponent`  least-squares slope of log risk against log step over the tail of a curve: the
                         scaling exponent the kappa sweeps compare.
* `tau_order_statistics` order statistics of a tau vector at ranks floor(1.1^k) from both tails (same sampling as
                         `adana_b200.logging.tau_stats.compute_tau_order_statistics`, which handles the LLM case).
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, Optional, Sequence

import numpy as np

from .plrf import PowerLawRF


def compare_rules(problem: PowerLawRF, rules: Dict[str, tuple], steps: int, batch: int, seed: int = 0,
                  eval_at: Optional[Sequence[int]] = None, on_eval: Optional[Callable] = None):
    """-> {"steps": array, name: risks array, ...}; `rules` maps a name to an `(init, update)` pair."""
    rng = np.random.default_rng(seed)
    if eval_at is None:
        eval_at = np.unique(np.round(np.geomspace(1, steps, 40)).astype(int))
    eval_set = set(int(e) for e in eval_at)
    w = {k: np.zeros(problem.d) for k in rules}
    st = {k: rules[k][0](w[k]) for k in rules}
    out = {k: [problem.population_risk(w[k])] for k in rules}
    ts = [0]
    for t in range(1, steps + 1):
        X, y = problem.sample(rng, batch)
        for k, (_, update) in rules.items():
            g = problem.batch_gradient(w[k], X, y)
            dw, st[k] = update(g, st[k], w[k])
            w[k] = w[k] + dw
        if t in eval_set:
            ts.append(t)
            for k in rules:
                out[k].append(problem.population_risk(w[k]))
            if on_eval is not None:
                on_eval(t, w, st)
    res = {k: np.array(v) for k, v in out.items()}
    res["steps"] = np.array(ts)
    res["_final_states"] = st
    return res


def sweep(problem: PowerLawRF, make_rule: Callable[[float], tuple], values: Iterable[float], steps: int, batch: int,
          seed: int = 0):
    """One curve per value of the swept hyper-parameter, all on the same batches."""
    rules = {f"{v:g}": make_rule(v) for v in values}
    return compare_rules(problem, rules, steps, batch, seed)


def final_risk_exponent(steps: np.ndarray, risks: np.ndarray, limit_risk: float = 0.0, tail: float = 0.5) -> float:
    """Slope of log(risk - limit_risk) against log(step) over the last `tail` fraction (in log-time) of the curve."""
    m = steps > 0
    s, r = np.log(steps[m]), risks[m] - limit_risk
    keep = (s >= s.max() - tail * (s.max() - s.min())) & (r > 0)
    if keep.sum() < 2:
        return float("nan")
    return float(np.polyfit(s[keep], np.log(r[keep]), 1)[0])


def tau_order_statistics(tau: np.ndarray, base: float = 1.1):
    """(largest-side, smallest-side) order statistics at ranks floor(base^k)."""
    t = np.sort(np.asarray(tau, dtype=np.float64).ravel())
    n = len(t)
    if n == 0:
        return np.array([]), np.array([])
    kmax = int(np.ceil(np.log(n) / np.log(base)))
    idx = np.unique(np.minimum((base ** np.arange(kmax + 1)).astype(np.int64) - 1, n - 1))
    return t[(n - 1) - idx], t[idx]
