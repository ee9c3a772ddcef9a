"""Drawings of the studies, one function per figure family, as SVG through `adana_b200.figures.LineChart` (no plotting
package).  Every function takes the output of the study function of the same name and a path, and returns the path.

Figure families and the reference script each stands in for:
  lr_law               bighead_lr_scaling.py   kept lrs per size, fitted law, bootstrap band
  curvature            lr_curvature_analysis.py   loss against lr per size with the fitted parabolas
  loss_laws            compare_scaling_rules*.py   final loss against compute per optimizer with the joint fit
  residuals            compute_formula_comparison.py / compute_formula_residuals.py   residual of each fit
  compute_multiplier   compare_scaling_rules_ep.py --plot-compute-gain   baseline compute / optimizer compute
  savings              compute_saved.py   compute saved against model compute with the fitted lines
  gamma3               gamma3_factor_scaling.py   best gamma_3_factor against iterations
  tau_cdf              plot_tau_summary.py, plot_aggregated_tensors.py   tau CDFs on the compressed-logit axis
  optimizer_stats      snr_clipping_plots.py   a logged statistic against tokens with its unclipped theory
  hoyer                hoyer_final_loss.py, hoyer_vs_regularization.py   final loss against the Hoyer coefficient
  hoyer_curves         hoyer_loss_curves.py   cross-entropy and Hoyer-term curves coloured by the coefficient
  kappa_curves / kappa_slice   llm_hummingbird_plot.py, llm_hummingbird_slice_plot.py
  size_curves          bighead_loss_curves.py   best run of each size, loss against compute
"""
from __future__ import annotations

from pathlib import Path
from typing import Dict, Optional, Sequence

import numpy as np

from ..figures import LineChart
from . import palette
from .loss_laws import broken, single
from .lr_law import confidence_band, predict
from .tau_cdf import PROB_TICKS, prob_axis


def lr_law(report: Dict, out, band_samples=None) -> Path:
    f = report["fit"]
    ch = LineChart(f"lr = {f['a']:.3g} ({f['b']:.3g} + P)^{f['d']:.3f}", "non-embedding parameters P",
                   "peak learning rate", logx=True, logy=True)
    P_all = []
    for size, d in report["sizes"].items():
        P = d["non_emb_params"]
        P_all.append(P)
        ch.add([P] * len(d["top_k_data"]), [t["lr"] for t in d["top_k_data"]], f"{size}", palette.viridis(len(P_all) / max(len(report["sizes"]), 1)),
               line=False)
        if d.get("others"):
            ch.add([P] * len(d["others"]), [t["lr"] for t in d["others"]], "", "#bbbbbb", line=False)
    grid = np.geomspace(min(P_all) / 2, max(P_all) * 4, 120)
    ch.add(grid, predict(grid, f["a"], f["b"], f["d"]), "fit", "#000000", dashed=True)
    if band_samples is not None:
        med, lo, hi = confidence_band(grid, *band_samples)
        ch.add(grid, lo, "95 % band", "#888888", opacity=0.6)
        ch.add(grid, hi, "", "#888888", opacity=0.6)
    return ch.save(out)


def curvature(report: Dict, table: Dict, out) -> Path:
    ch = LineChart("loss against learning rate with the fitted parabolas", "learning rate", "final validation loss", logx=True)
    n = max(len(report["per_size"]), 1)
    for i, (size, d) in enumerate(report["per_size"].items()):
        col = palette.viridis(i / n)
        rows = sorted(table[int(size)], key=lambda r: r["lr"])
        lrs = np.array([r["lr"] for r in rows])
        ch.add(lrs, [r["val_loss"] for r in rows], f"{size} (κ={d['kappa']:.3g})", col, line=False)
        if np.isfinite(d["kappa"]):
            g = np.geomspace(lrs.min(), lrs.max(), 60)
            ch.add(g, d["L_star"] + d["kappa"] * (np.log(g) - np.log(d["lr_star"])) ** 2, "", col, opacity=0.7)
    return ch.save(out)


def loss_laws(curves: Sequence[Dict], fit: Dict, out, metric: str = "compute (PFLOP-hours)") -> Path:
    """curves: [{name, compute, loss}], fit: the output of `loss_laws.fit_joint`."""
    ch = LineChart(f"loss against {metric}; shared floor a = {fit['a']:.3f}", metric, "final validation loss", logx=True, logy=True)
    for d in curves:
        col = palette.color(d["name"].split("_")[0], None) or None
        C = np.asarray(d["compute"], dtype=np.float64)
        ch.add(C, d["loss"], palette.display_name(d["name"]), col, line=False)
        q = fit["curves"].get(d["name"])
        if q:
            g = np.geomspace(C.min() / 2, C.max() * 2, 100)
            y = broken(g, fit["a"], q["b"], q["c"], q["e"], q["f"]) if "e" in q else single(g, fit["a"], q["b"], q["c"])
            ch.add(g, y, "", ch.series[-1]["color"], dashed=True, opacity=0.7)
    return ch.save(out)


def residuals(fits: Dict[str, Dict], compute, out) -> Path:
    """fits: label -> a report of fit_single / fit_broken over the same `compute` points."""
    ch = LineChart("residuals of the loss-law fits", "compute (PFLOP-hours)", "loss - fit", logx=True)
    for label, f in fits.items():
        ch.add(compute, f["residuals"], f"{label} (R²={f['r_squared']:.4f})", markers=True)
    ch.hline(0.0, "", "#000000")
    return ch.save(out)


def compute_multiplier(series: Dict[str, tuple], out, baseline: str = "adamw") -> Path:
    """series: optimizer -> (compute, multiplier) from `multiplier_piecewise` or `multiplier_from_fits`."""
    ch = LineChart(f"compute multiplier over {palette.display_name(baseline)}", "compute (PFLOP-hours)",
                   "baseline compute at equal loss / compute", logx=True)
    for name, (C, g) in series.items():
        ch.add(C, g, palette.display_name(name), palette.color(name, None), markers=True, dashed=palette.linestyle(name) == "--")
    ch.hline(1.0, palette.display_name(baseline), palette.color(baseline))
    return ch.save(out)


def savings(datasets: Sequence[Dict], lines: Dict, out) -> Path:
    ch = LineChart("compute saved against the baseline", "model compute (PFLOP-hours)", "compute saved (PFLOP-hours)", logx=True, logy=True)
    for d in datasets:
        x = np.asarray(d["x"], dtype=np.float64)
        ch.add(x, d["y"], palette.display_name(d["name"]), palette.color(d["name"], None), line=False)
        q = lines["curves"].get(d["name"])
        if q:
            g = np.geomspace(x.min(), x.max(), 50)
            ch.add(g, q["b"] * g ** q["c"], f"{q['b']:.3g} X^{q['c']:.2f}", ch.series[-1]["color"], dashed=True)
    return ch.save(out)


def gamma3(report: Dict, out) -> Path:
    from .gamma3 import evaluate

    ch = LineChart("best gamma_3_factor against training length", "iterations", "gamma_3_factor", logx=True, logy=True)
    sizes = sorted({p["size"] for p in report["points"]})
    for i, s in enumerate(sizes):
        pts = [p for p in report["points"] if p["size"] == s]
        ch.add([p["iterations"] for p in pts], [p["gamma_3_factor"] for p in pts], f"{s} heads",
               palette.viridis(i / max(len(sizes) - 1, 1)), line=False)
    if report["params"]:
        T = np.array([p["iterations"] for p in report["points"]], dtype=np.float64)
        g = np.geomspace(T.min(), T.max(), 60)
        a, b = report["params"]
        ch.add(g, evaluate(g, report["params"], report["kind"]), f"{report['kind']}: {a:.3g}, {b:.3g}", "#000000", dashed=True)
    return ch.save(out)


def tau_cdf(group: Dict, out, title: str = "", raw: bool = False) -> Path:
    """group: one entry of `tau_cdf.summary(...)["groups"]` or of `all_kinds`."""
    ticks = [(float(prob_axis(p)[0]), f"{100 * p:g}%") for p in PROB_TICKS]
    ch = LineChart(title or f"tau CDF ({group['tensors']} tensors)", "tau" if raw else "regularised tau",
                   "cumulative probability", logx=True, yticks=ticks)
    n = max(len(group["lines"]), 1)
    for i, ln in enumerate(group["lines"]):
        ch.add(ln["tau"], ln["y"], f"iter={ln['iteration']} (eval {ln['eval_step']})", palette.viridis(0.9 * i / n))
    return ch.save(out)


def optimizer_stats(stats: Dict[str, Dict], key: str, out) -> Path:
    d = stats[key]
    ch = LineChart(key, "tokens", key.split("/", 1)[-1], logx=True, logy=True)
    ch.add(d["tokens"], d["value"], "logged")
    if "theory" in d:
        ch.add(d["tokens"], d["theory"], "unclipped theory", "#000000", dashed=True)
    return ch.save(out)


def hoyer(by_coeff: Dict, out) -> Path:
    """by_coeff: the output of `sweeps.hoyer_loss_by_coefficient`; the coefficient 0 is drawn at a tenth of the
    smallest positive one so that it has a place on the log axis."""
    ch = LineChart("final loss against the Hoyer coefficient", "Hoyer coefficient (0 drawn at the left edge)",
                   "final validation loss", logx=True)
    pos = [p["hoyer_coeff"] for pts in by_coeff.values() for p in pts if p["hoyer_coeff"] > 0]
    zero_at = min(pos) / 10 if pos else 1e-6
    for (heads, opt), pts in sorted(by_coeff.items()):
        ch.add([p["hoyer_coeff"] or zero_at for p in pts], [p["final_val_loss"] for p in pts],
               f"{palette.display_name(opt)}, {heads} heads", palette.color(opt, None), markers=True)
    return ch.save(out)


def hoyer_curves(curves: Sequence[Dict], out, which: str = "loss") -> Path:
    """curves: the output of `sweeps.hoyer_curves`; `which` = "loss" (cross-entropy) or "hoyer" (the regulariser's own
    value).  Lines are coloured by the logarithm of the coefficient, the unregularised run is black."""
    x_key = "pf_days" if which == "loss" else "hoyer_pf_days"
    ch = LineChart("validation loss" if which == "loss" else "Hoyer term", "compute (PetaFLOP-days)", which, logx=True, logy=True)
    pos = [c["hoyer_coeff"] for c in curves if c["hoyer_coeff"] > 0]
    lo, hi = (min(pos), max(pos)) if pos else (1.0, 1.0)
    for c in curves:
        if not c[which]:
            continue
        col = "#000000" if c["hoyer_coeff"] <= 0 else palette.log_scale_color(c["hoyer_coeff"], lo, hi)
        ch.add(c[x_key], c[which], f"{palette.hoyer_label(c['hoyer_coeff'])} ({palette.display_name(c['opt'])})", col,
               dashed=palette.hoyer_linestyle(c["hoyer_coeff"]) != "-")
    return ch.save(out)


def kappa_curves(sweep: Dict, out, baseline: Optional[Dict] = None, kappa_min: float = 0.0) -> Path:
    ch = LineChart("validation loss for every kappa and clip-SNR", "training step", "validation loss", logy=True)
    seen = set()
    for (clip, kappa), v in sorted(sweep.items()):
        if kappa < kappa_min:
            continue
        op, w = palette.line_emphasis(kappa, kappa_min)
        label = "" if clip in seen else f"clipsnr={clip:g}"
        seen.add(clip)
        ch.add(v["steps"], v["losses"], label, palette.clipsnr_color(clip), opacity=op, width=w)
    if baseline:
        ch.add(baseline["steps"], baseline["losses"], "AdamW (baseline)", "#000000", dashed=True, width=3)
    return ch.save(out)


def kappa_slice(slices: Dict, out, baseline: Optional[Dict] = None) -> Path:
    ch = LineChart("final loss against kappa", "kappa", "final validation loss")
    for clip, d in sorted(slices.items()):
        ch.add(d["kappa"], d["final"], "ADANA" if clip >= 100 else f"DANA-MK4 (c={clip:g})", palette.clipsnr_color(clip), markers=True)
    if baseline:
        ch.hline(baseline["final"], "AdamW (baseline)", "#000000")
    return ch.save(out)


def size_curves(best: Dict[int, Dict], out, opt: str = "") -> Path:
    ch = LineChart(f"{palette.display_name(opt)}: best run of every size", "compute (PFLOP-hours)", "validation loss", logx=True, logy=True)
    n = max(len(best) - 1, 1)
    for i, (size, d) in enumerate(sorted(best.items())):
        ch.add(d["compute"], d["loss"], f"{size}: {d['final_loss']:.3f}", palette.viridis(i / n))
    return ch.save(out)
