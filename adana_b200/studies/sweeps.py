"""Studies that are selections over the run table rather than fits: the best run of every size with its loss curve
against compute, the GPU-hours ledger, the optimizer's logged schedule statistics against their unclipped theory, the
Hoyer-regularisation sweeps, and the kappa / clip-SNR sweep of one model size ("LLM hummingbird").

Reference scripts: visualization/bighead_loss_curves.py:194-390 (best run per size, FLOPs = 6 * non_emb * tokens),
compute_gpu_hours.py:223-545 (mean iter_dt x iterations x GPUs / 3600, best run per size, CSV), snr_clipping_plots.py:
115-190 (the four `optimizer/*` statistics with (1+t)^(1-kappa) and mfac (1+t)^(1-kappa)), hoyer_final_loss.py:146-327,
hoyer_loss_curves.py:114-300, hoyer_vs_regularization.py:76-227, llm_hummingbird_plot.py:92-178 and
llm_hummingbird_slice_plot.py:174-257 (final loss against kappa per clip-SNR, AdamW as a horizontal line).
"""
from __future__ import annotations

import csv
import math
from typing import Dict, Iterable, List, Optional, Sequence

import numpy as np

from .runs import Run, select
from .sizes import PF_DAY, PFH, model_size, size_key


# ---- best run per size, loss against compute -----------------------------------------------------------------------
def best_runs_per_size(runs: Iterable[Run], rule: str, opt: Optional[str] = None, key: str = "val/loss", **sel) -> Dict[int, Dict]:
    """size -> {run, final_loss, compute (PFH per record), loss (per record)} of the finished run with the lowest final
    validation loss.  Compute of a record is 6 * non_emb * tokens seen."""
    best: Dict[int, Run] = {}
    for r in select(runs, opt=opt, **sel):
        size, loss = r.config.get(size_key(rule)), r.final_val_loss
        if size is None or loss is None:
            continue
        if int(size) not in best or loss < best[int(size)].final_val_loss:
            best[int(size)] = r
    out = {}
    for size, r in sorted(best.items()):
        m = model_size(size, rule)
        toks, losses = r.series(key, x="tokens")
        out[size] = {"run": r.name, "final_loss": r.final_val_loss, "non_emb": m.non_emb,
                     "compute": [6.0 * m.non_emb * t / PFH for t in toks], "loss": list(losses)}
    return out


# ---- GPU hours ------------------------------------------------------------------------------------------------------------
def format_params(n: Optional[float]) -> str:
    if not n:
        return "N/A"
    for div, unit in ((1e9, "B"), (1e6, "M"), (1e3, "K")):
        if n >= div:
            return f"{n / div:.2f}{unit}" if unit == "B" else f"{n / div:.1f}{unit}"
    return str(int(n))


def gpu_hours_rows(runs: Iterable[Run], rule: Optional[str] = None, opt: Optional[str] = None) -> List[Dict]:
    """One row per run that carries timing: mean `iter_dt` (from the history, else the summary's `iter_dt`, else
    `_runtime` / iterations) x iterations done x world size / 3600."""
    rows = []
    for r in select(runs, opt=opt, finished=False, need=()):
        done = r.summary.get("iter", 0) or 0
        total = done if done > 0 else (r.config.get("iterations", 0) or 0)
        _, dts = r.series("iter_dt")
        dts = [d for d in dts if d is not None and math.isfinite(d)]
        if dts:
            mean = sum(dts) / len(dts)
        elif r.summary.get("iter_dt"):
            mean = float(r.summary["iter_dt"])
        elif r.summary.get("_runtime") and done > 0:
            mean = float(r.summary["_runtime"]) / done
        else:
            continue
        world = int(r.config.get("world_size", 1) or 1)
        size = r.config.get(size_key(rule)) if rule else r.config.get("n_head")
        total_params = model_size(size, rule).total_params if rule and size is not None else None
        wall = mean * total
        gpu = next((str(v) for k, v in {**r.config, **r.summary}.items() if "gpu" in k.lower() and isinstance(v, str)), None)
        rows.append({"run_name": r.name, "size": size, "total_params": total_params, "world_size": world,
                     "total_iterations": total, "iter_dt_mean": mean, "wall_time_hours": wall / 3600.0,
                     "gpu_hours": wall * world / 3600.0, "gpu_type": gpu, "final_loss": r.final_val_loss})
    return rows


def gpu_hours_by_size(rows: Sequence[Dict]) -> List[Dict]:
    """The lowest-loss run of every size (the first one when none has a loss), smallest model first."""
    groups: Dict = {}
    for r in rows:
        groups.setdefault(r["size"], []).append(r)
    out = []
    for size, g in groups.items():
        with_loss = [r for r in g if r["final_loss"] is not None]
        b = min(with_loss, key=lambda r: r["final_loss"]) if with_loss else g[0]
        out.append({**b, "model_size_formatted": format_params(b["total_params"]) if b["total_params"] else f"size={size}",
                    "num_runs": len(g)})
    return sorted(out, key=lambda r: (r["total_params"] is None, r["total_params"] or 0, r["size"] or 0))


def gpu_hours_table(rows: Sequence[Dict], title: str = "GPU Hours by Model Size") -> str:
    lines = [title, f"{'Model Size':<15} {'GPU Hours':<12} {'Wall Time (h)':<15} {'GPUs':<8} {'Iters':<12} {'iter_dt (s)':<12} {'GPU Type':<20}",
             "-" * 100]
    for r in rows:
        lines.append(f"{r['model_size_formatted']:<15} {r['gpu_hours']:<12.1f} {r['wall_time_hours']:<15.2f} "
                     f"{r['world_size']:<8} {r['total_iterations']:<12} {r['iter_dt_mean']:<12.4f} {str(r['gpu_type'] or 'N/A')[:18]:<20}")
    lines += ["-" * 100, f"{'Total':<15} {sum(r['gpu_hours'] for r in rows):<12.1f}"]
    return "\n".join(lines)


def write_csv(rows: Sequence[Dict], path) -> None:
    if not rows:
        return
    with open(path, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=list(rows[0]))
        w.writeheader()
        w.writerows(rows)


# ---- logged optimizer statistics against their theory ------------------------------------------------------------------
SCHEDULE_STATS = ("optimizer/m_norm", "optimizer/kappa_factor_schedule", "optimizer/auto_factor", "optimizer/alpha_schedule")


def optimizer_statistics(run: Run, kappa: Optional[float] = None) -> Dict[str, Dict]:
    """Per statistic: tokens, value (positive finite records, by tokens) and, where there is one, the unclipped theory:
    (1+t)^(1-kappa) for the kappa factor and mfac (1+t)^(1-kappa) for the momentum coefficient; the gap between the
    logged coefficient and its theory line is what SNR clipping removes."""
    kappa = run.config.get("kappa", 0.85) if kappa is None else kappa
    out = {}
    for key in SCHEDULE_STATS:
        rows = [r for r in run.history(["tokens", "iter", key]) if r["tokens"] > 0 and r["iter"] > 0
                and r[key] > 0 and math.isfinite(r[key])]
        rows.sort(key=lambda r: r["tokens"])
        if not rows:
            continue
        t = np.array([r["iter"] for r in rows], dtype=np.float64)
        entry = {"tokens": np.array([r["tokens"] for r in rows], dtype=np.float64),
                 "value": np.array([r[key] for r in rows], dtype=np.float64), "iter": t}
        if key == "optimizer/kappa_factor_schedule":
            entry["theory"] = (1 + t) ** (1 - kappa)
        elif key == "optimizer/alpha_schedule":
            mfac = np.array([r.get("optimizer/auto_factor", math.nan) for r in rows], dtype=np.float64)
            if np.isfinite(mfac).all():
                entry["theory"] = mfac * (1 + t) ** (1 - kappa)
        out[key] = entry
    return out


# ---- Hoyer sweeps -----------------------------------------------------------------------------------------------------------
def hoyer_points(runs: Iterable[Run], heads: Optional[Sequence[int]] = None, opts: Optional[Sequence[str]] = None,
                 batch_tokens: Optional[int] = None) -> List[Dict]:
    """One row per finished run of a Qwen3 Hoyer sweep: heads, optimizer, coefficient, final validation loss, final
    Hoyer value (`train/hoyer_loss` or `val/hoyer_loss` when logged), compute in PetaFLOP-days."""
    rows = []
    for r in select(runs, need=()):
        h, o = r.config.get("n_head"), r.opt
        if r.final_val_loss is None or h is None or (heads and h not in heads) or (opts and o not in opts):
            continue
        m = model_size(h, "Qwen3_Hoyer")
        its = r.summary.get("iter") or r.config.get("iterations") or 0
        per_it = batch_tokens or (r.config.get("batch_size", 1) * r.config.get("acc_steps", 1) * r.config.get("sequence_length", 512))
        rows.append({"run": r.name, "heads": int(h), "opt": o, "hoyer_coeff": float(r.config.get("hoyer_loss_coeff", 0.0) or 0.0),
                     "final_val_loss": float(r.final_val_loss),
                     "hoyer_value": r.summary.get("val/hoyer_loss", r.summary.get("train/hoyer_loss")),
                     "pf_days": 6.0 * m.non_emb * per_it * its / PF_DAY})
    return rows


def hoyer_curves(runs: Iterable[Run], heads: Optional[int] = None, opt: Optional[str] = None, key: str = "val/loss",
                 hoyer_key: str = "train/hoyer_loss") -> List[Dict]:
    """Per finished run of a Hoyer sweep: its coefficient, the cross-entropy curve and, where logged, the curve of the
    Hoyer term itself, both against compute in PetaFLOP-days; sorted by coefficient (the figures colour by it)."""
    out = []
    for r in select(runs, opt=opt, need=()):
        h = r.config.get("n_head")
        if h is None or (heads is not None and h != heads):
            continue
        m = model_size(h, "Qwen3_Hoyer")
        per_tok = 6.0 * m.non_emb / PF_DAY
        toks, ce = r.series(key, x="tokens")
        if not ce:
            continue
        toks_h, hv = r.series(hoyer_key, x="tokens")
        out.append({"run": r.name, "heads": int(h), "opt": r.opt, "hoyer_coeff": float(r.config.get("hoyer_loss_coeff", 0.0) or 0.0),
                    "pf_days": [per_tok * t for t in toks], "loss": list(ce),
                    "hoyer_pf_days": [per_tok * t for t in toks_h], "hoyer": list(hv)})
    return sorted(out, key=lambda d: d["hoyer_coeff"])


def hoyer_loss_by_coefficient(points: Sequence[Dict]) -> Dict:
    """(heads, opt) -> coefficients ascending with the best final loss at each."""
    g: Dict = {}
    for p in points:
        cur = g.setdefault((p["heads"], p["opt"]), {})
        c = p["hoyer_coeff"]
        if c not in cur or p["final_val_loss"] < cur[c]["final_val_loss"]:
            cur[c] = p
    return {k: [v[c] for c in sorted(v)] for k, v in g.items()}


# ---- kappa / clip-SNR sweep at one size ---------------------------------------------------------------------------------------
def kappa_sweep(runs: Iterable[Run], n_head: int, opts: Sequence[str] = ("dana-star-mk4", "dana-mk4", "adana", "dana-star"),
                key: str = "val/loss") -> Dict:
    """(clipsnr, kappa) -> {steps, losses, final} of the finished runs of one size; runs without a clip-SNR (the
    unclipped optimizers) are filed under clipsnr 100."""
    out: Dict = {}
    for r in select(runs, need=("kappa",)):
        if r.opt not in opts or r.config.get("n_head") != n_head:
            continue
        clip = r.config.get("clipsnr")
        clip = 100.0 if clip in (None, "None") or r.opt in ("adana", "dana-star") else float(clip)
        steps, losses = r.series(key)
        k = (clip, round(float(r.config["kappa"]), 4))
        if losses and (k not in out or losses[-1] < out[k]["final"]):
            out[k] = {"steps": list(steps), "losses": list(losses), "final": float(losses[-1]), "run": r.name}
    return out


def adamw_baseline(runs: Iterable[Run], n_head: int, key: str = "val/loss") -> Optional[Dict]:
    best = None
    for r in select(runs, opt="adamw", need=()):
        if r.config.get("n_head") != n_head:
            continue
        steps, losses = r.series(key)
        if losses and (best is None or losses[-1] < best["final"]):
            best = {"steps": list(steps), "losses": list(losses), "final": float(losses[-1]), "run": r.name}
    return best


def on_tenths_grid(kappa: float) -> bool:
    """False for the half-step values (0.05, 0.15, ...) that only some clip-SNR settings were run at."""
    return round(round(kappa * 100) / 100 * 100) % 10 != 5


def kappa_slices(sweep: Dict, kappa_min: float = 0.0, tenths_only: bool = True) -> Dict[float, Dict[str, List[float]]]:
    """clipsnr -> {kappa: [...], final: [...]}: the final loss as a function of kappa, one line per clip-SNR."""
    out: Dict[float, Dict[str, List[float]]] = {}
    for (clip, kappa), v in sorted(sweep.items()):
        if kappa >= kappa_min and (on_tenths_grid(kappa) or not tenths_only):
            d = out.setdefault(clip, {"kappa": [], "final": []})
            d["kappa"].append(kappa)
            d["final"].append(v["final"])
    return out
