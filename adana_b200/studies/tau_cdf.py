"""Distribution of the Dana-Star tau estimates, rebuilt from the sparse order statistics a run stores.

`logging/tau_stats.py` keeps, per parameter tensor and collection time, the floor(1.1^k)-th smallest and largest tau
values.  Each stored value is one point of the tensor's empirical CDF (the j-th smallest of n sits at (j+1)/n, the j-th
largest at (n-j)/n); tensors of one kind (all blocks' `mlp.c_fc.weight`, say) are merged by interpolating their CDFs on
the union of their tau values and averaging.  For plotting, tau is optionally regularised the way the optimizer does
(tau_reg = max(min(tau, 1/2) / (1 - min(tau, 1/2)), 1/(1+t))) and probabilities go on a logit axis whose two tails,
below 0.1 % and above 99.9 %, are squeezed into one unit each so that 0 and 1 stay finite.

Reference: visualization/plot_aggregated_tensors.py:26-330, 410-440 and plot_tau_summary.py (the 2 x 2 summary of
embedding, attention, MLP and output tensors at four times of training).
"""
from __future__ import annotations

import json
import math
import pickle
import re
from collections import defaultdict
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

_BLOCK = re.compile(r"\.h\.\d+\.")
_LO, _HI = 0.001, 0.999
SUMMARY_GROUPS = {"Embedding": "Transformer wte.weight", "Attention": "Transformer attn.c_attn.weight",
                  "MLP": "Transformer mlp.c_fc.weight", "Output": "Transformer module.lm_head.weight"}


def regularize_tau(tau, t):
    c = np.minimum(np.asarray(tau, dtype=np.float64), 0.5)
    return np.maximum(c / (1.0 - c), 1.0 / (1.0 + t))


def prob_axis(prob):
    """Probability -> axis position: log10 odds inside [0.1 %, 99.9 %]; [0, 0.1 %] maps linearly onto the unit below
    log10 odds(0.1 %), [99.9 %, 1] onto the unit above log10 odds(99.9 %)."""
    p = np.atleast_1d(np.asarray(prob, dtype=np.float64))
    y_hi, y_lo = math.log10(_HI / (1 - _HI)), math.log10(_LO / (1 - _LO))
    y = np.zeros_like(p)
    low, high = p < _LO, p > _HI
    mid = ~low & ~high
    y[low] = y_lo - 1 + p[low] / _LO
    pm = np.clip(p[mid], 1e-10, 1 - 1e-10)
    y[mid] = np.log10(pm / (1 - pm))
    y[high] = y_hi + (p[high] - _HI) / (1 - _HI)
    return y


PROB_TICKS = [0.001, 0.01, 0.1, 0.5, 0.9, 0.99, 0.999, 1.0]


def stored_ranks(n: int, count: int) -> np.ndarray:
    """0-based ranks of the first `count` stored order statistics of a tensor with n elements."""
    kmax = int(math.ceil(math.log(n * 10) / math.log(1.1)))
    r = np.unique(np.int32(1.1 ** np.arange(kmax + 1)) - 1)
    return r[r < n][:count]


def cdf_from_order_stats(smallest, largest, n: int) -> Tuple[np.ndarray, np.ndarray]:
    """-> (tau values ascending, P(tau <= value)) from one tensor's stored statistics."""
    smallest, largest = np.asarray(smallest, dtype=np.float64), np.asarray(largest, dtype=np.float64)
    if len(smallest) == 0 and len(largest) == 0:
        return np.array([]), np.array([])
    ranks = stored_ranks(n, max(len(smallest), len(largest)))
    ks, kl = min(len(smallest), len(ranks)), min(len(largest), len(ranks))
    tau = np.concatenate([smallest[:ks], largest[:kl]])
    cdf = np.concatenate([(ranks[:ks] + 1) / n, (n - ranks[:kl]) / n])
    order = np.argsort(tau, kind="stable")
    return tau[order], cdf[order]


def merge_cdfs(cdfs: Sequence[Tuple[np.ndarray, np.ndarray]]) -> Dict[str, np.ndarray]:
    """Mean of several CDFs on the union of their support points (0 left of a CDF's first point, 1 right of its last)."""
    if not cdfs:
        return {"tau_values": np.array([]), "cdf_values": np.array([])}
    grid = np.unique(np.concatenate([t for t, _ in cdfs]))
    return {"tau_values": grid,
            "cdf_values": np.mean([np.interp(grid, t, c, left=0.0, right=1.0) for t, c in cdfs], axis=0)}


def kind_of(param_name: str) -> str:
    """`module.transformer.h.3.mlp.c_fc.weight` -> `Transformer mlp.c_fc.weight`: the block index and the wrapper
    prefix go, so that all blocks' tensors of one kind share a name."""
    return "Transformer " + _BLOCK.sub(".", param_name).replace("module.transformer.", "")


def group_by_kind(param_names: Sequence[str]) -> Dict[str, List[str]]:
    groups = defaultdict(list)
    for p in param_names:
        groups[kind_of(p)].append(p)
    return dict(groups)


def load_directory(tau_stats_dir):
    """-> (metadata, {iteration: stored record}, sorted iterations) of a run's `tau_stats/` folder."""
    d = Path(tau_stats_dir)
    meta = json.loads((d / "tau_stats_metadata.json").read_text())
    data = {}
    for f in sorted(d.glob("tau_stats_iter_*.pkl")):
        with open(f, "rb") as fh:
            rec = pickle.load(fh)
        data[rec["metadata"]["iteration"]] = rec
    return meta, data, sorted(data)


def group_cdf(record: Dict, params: Sequence[str], iteration: Optional[int] = None, raw: bool = False):
    """Merged CDF of the tensors `params` in one stored record -> (tau or tau_reg, probability, axis position)."""
    parts = []
    for p in params:
        st = record["tau_statistics"].get(p)
        if st is None:
            continue
        t, c = cdf_from_order_stats(st["smallest_order_stats"], st["largest_order_stats"], st["num_elements"])
        if len(t):
            parts.append((t, c))
    m = merge_cdfs(parts)
    tau = m["tau_values"]
    if not raw and len(tau):
        tau = regularize_tau(tau, record["metadata"]["iteration"] if iteration is None else iteration)
    return tau, m["cdf_values"], prob_axis(m["cdf_values"]) if len(tau) else np.array([])


def four_times(iterations: Sequence[int]) -> List[int]:
    """Early, one third, two thirds and last of the collection times."""
    n = len(iterations)
    return [iterations[0], iterations[n // 3], iterations[2 * n // 3], iterations[-1]]


def summary(tau_stats_dir, raw: bool = False, groups: Optional[Dict[str, str]] = None) -> Dict:
    """{display name: {"tensors": k, "lines": [{iteration, eval_step, tau, prob, y}]}} for the four summary kinds (any
    of them that the model has; with the bare parameter names this framework logs, `lm_head.weight` and
    `transformer.*` are matched as well)."""
    meta, data, its = load_directory(tau_stats_dir)
    names = sorted(data[its[0]]["tau_statistics"])
    by_kind = group_by_kind(names)
    out = {"metadata": meta, "iterations": four_times(its), "groups": {}}
    for disp, key in (groups or SUMMARY_GROUPS).items():
        params = by_kind.get(key)
        if params is None:     # names logged without the DDP prefix
            params = [n for n in names if kind_of("module." + n) == key or kind_of("module.transformer." + n) == key]
        if not params:
            continue
        lines = []
        for it in out["iterations"]:
            tau, prob, y = group_cdf(data[it], params, raw=raw)
            lines.append({"iteration": it, "eval_step": data[it]["metadata"].get("eval_step_number"),
                          "tau": tau, "prob": prob, "y": y})
        out["groups"][disp] = {"tensors": len(params), "lines": lines}
    return out


def all_kinds(tau_stats_dir, raw: bool = False, iterations: Optional[Sequence[int]] = None) -> Dict:
    """One merged CDF per kind of tensor and chosen collection time (default: all)."""
    meta, data, its = load_directory(tau_stats_dir)
    use = [i for i in (iterations or its) if i in data]
    by_kind = group_by_kind(sorted(data[its[0]]["tau_statistics"]))
    out = {"metadata": meta, "iterations": use, "groups": {}}
    for kind, params in sorted(by_kind.items()):
        lines = []
        for it in use:
            tau, prob, y = group_cdf(data[it], params, raw=raw)
            lines.append({"iteration": it, "eval_step": data[it]["metadata"].get("eval_step_number"),
                          "tau": tau, "prob": prob, "y": y})
        out["groups"][kind] = {"tensors": len(params), "lines": lines}
    return out
