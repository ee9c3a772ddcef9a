"""Figure scripts: training curves, loss against compute, the learning-rate scaling law, the kappa sweep
("hummingbird") and the tau order statistics, drawn headless to SVG files.

The reference's `visualization/` tree pulls runs from the W&B API and draws matplotlib figures
(compare_scaling_rules.py, bighead_loss_curves.py, bighead_lr_scaling.py, compute_saved.py, llm_hummingbird.py,
plot_tau_summary.py, jax/hummingbird_plot.py, jax/taustats_plot_from_data.py).  Here the inputs are the files
this framework writes itself (`<exp>/metrics.jsonl`, the JSON of `adana_b200.theory.generate`) and the
numbers come from `adana_b200.analysis`; the drawing needs no plotting package: `LineChart` writes plain SVG
(linear or log axes, legend, markers), so the scripts run on a training node.

    python -m adana_b200.figures curves  <exp_dir> [<exp_dir> ...] --out curves.svg [--key val/loss]
    python -m adana_b200.figures compute <exp_dir>:<non_emb> [...]  --out compute.svg
    python -m adana_b200.figures lr-law  sizes.json --out lr_law.svg        # {"P": [...], "lr": [...]}
    python -m adana_b200.figures hummingbird hummingbird.json --out hummingbird.svg
    python -m adana_b200.figures hummingbird-multi mk4.json ademamix.json --out hummingbird_all.svg
    python -m adana_b200.figures taustats    taustats.json    --out taustats.svg
"""
from __future__ import annotations

import argparse
import html
import json
import math
from pathlib import Path
from typing import List, Optional, Sequence

import numpy as np

PALETTE = ["#1f77b4", "#d62728", "#2ca02c", "#ff7f0e", "#9467bd", "#8c564b", "#17becf", "#7f7f7f", "#bcbd22", "#e377c2"]


class LineChart:
    """A small SVG line chart: `add(x, y, label)` any number of series, then `save(path)`."""

    def __init__(self, title="", xlabel="", ylabel="", logx=False, logy=False, width=760, height=480, yticks=None):
        self.title, self.xlabel, self.ylabel, self.logx, self.logy = title, xlabel, ylabel, logx, logy
        self.w, self.h = width, height
        self.series: List[dict] = []
        self.yticks = yticks            # [(position, label)] in place of the computed ticks (transformed axes)

    def add(self, x, y, label="", color=None, markers=False, dashed=False, line=True, opacity=1.0, width=1.6):
        x, y = np.asarray(x, dtype=np.float64), np.asarray(y, dtype=np.float64)
        ok = np.isfinite(x) & np.isfinite(y)
        if self.logx:
            ok &= x > 0
        if self.logy:
            ok &= y > 0
        self.series.append(dict(x=x[ok], y=y[ok], label=label, color=color or PALETTE[len(self.series) % len(PALETTE)],
                                markers=markers, dashed=dashed, line=line, opacity=opacity, width=width))
        return self

    def hline(self, y, label="", color="#888888", dashed=True):
        """Horizontal line across the range of the series added so far."""
        have = [s["x"] for s in self.series if len(s["x"])]
        xs = np.concatenate(have) if have else np.array([1.0 if self.logx else 0.0, 10.0 if self.logx else 1.0])
        return self.add([xs.min(), xs.max()], [y, y], label, color, dashed=dashed)

    @staticmethod
    def _ticks(lo, hi, log):
        if log:
            a, b = math.floor(math.log10(lo)), math.ceil(math.log10(hi))
            return [10.0 ** k for k in range(a, b + 1)]
        span = hi - lo or 1.0
        step = 10 ** math.floor(math.log10(span / 5))
        for m in (1, 2, 5, 10):
            if span / (step * m) <= 8:
                step *= m
                break
        first = math.ceil(lo / step) * step
        return [first + i * step for i in range(int((hi - first) / step) + 1)]

    def svg(self) -> str:
        pts = [s for s in self.series if len(s["x"])]
        if not pts:
            raise ValueError("nothing to draw")
        tx = (lambda v: np.log10(v)) if self.logx else (lambda v: v)
        ty = (lambda v: np.log10(v)) if self.logy else (lambda v: v)
        xs = np.concatenate([s["x"] for s in pts])
        ys = np.concatenate([s["y"] for s in pts])
        x0, x1, y0, y1 = xs.min(), xs.max(), ys.min(), ys.max()
        if x0 == x1:
            x0, x1 = x0 * 0.9 - 1e-12, x1 * 1.1 + 1e-12
        if y0 == y1:
            y0, y1 = y0 * 0.9 - 1e-12, y1 * 1.1 + 1e-12
        L, R, T, B = 70, 170, 36, 52
        pw, ph = self.w - L - R, self.h - T - B
        fx = lambda v: L + (tx(v) - tx(x0)) / (tx(x1) - tx(x0)) * pw
        fy = lambda v: T + ph - (ty(v) - ty(y0)) / (ty(y1) - ty(y0)) * ph
        out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{self.w}" height="{self.h}" font-family="sans-serif" font-size="12">',
               f'<rect width="{self.w}" height="{self.h}" fill="white"/>',
               f'<rect x="{L}" y="{T}" width="{pw}" height="{ph}" fill="none" stroke="#333"/>',
               f'<text x="{L + pw / 2}" y="20" text-anchor="middle" font-size="14">{html.escape(self.title)}</text>',
               f'<text x="{L + pw / 2}" y="{self.h - 12}" text-anchor="middle">{html.escape(self.xlabel)}</text>',
               f'<text x="16" y="{T + ph / 2}" text-anchor="middle" transform="rotate(-90 16 {T + ph / 2})">{html.escape(self.ylabel)}</text>']
        fmt = lambda v: f"{v:.3g}"
        for t in self._ticks(x0, x1, self.logx):
            if x0 <= t <= x1:
                out.append(f'<line x1="{fx(t):.1f}" y1="{T}" x2="{fx(t):.1f}" y2="{T + ph}" stroke="#ddd"/>')
                out.append(f'<text x="{fx(t):.1f}" y="{T + ph + 16}" text-anchor="middle">{fmt(t)}</text>')
        for t, lab in (self.yticks or [(t, fmt(t)) for t in self._ticks(y0, y1, self.logy)]):
            if y0 <= t <= y1:
                out.append(f'<line x1="{L}" y1="{fy(t):.1f}" x2="{L + pw}" y2="{fy(t):.1f}" stroke="#ddd"/>')
                out.append(f'<text x="{L - 6}" y="{fy(t) + 4:.1f}" text-anchor="end">{html.escape(str(lab))}</text>')
        for i, s in enumerate(pts):
            d = " ".join(f"{fx(a):.1f},{fy(b):.1f}" for a, b in zip(s["x"], s["y"]))
            dash = ' stroke-dasharray="6 4"' if s["dashed"] else ""
            if s["line"]:
                out.append(f'<polyline points="{d}" fill="none" stroke="{s["color"]}" stroke-width="{s["width"]:.2g}" '
                           f'stroke-opacity="{s["opacity"]:.2g}"{dash}/>')
            if s["markers"] or not s["line"]:
                out += [f'<circle cx="{fx(a):.1f}" cy="{fy(b):.1f}" r="3" fill="{s["color"]}"/>' for a, b in zip(s["x"], s["y"])]
            if not s["label"]:
                continue
            ly = T + 14 + 18 * sum(1 for q in pts[:i] if q["label"])
            out.append(f'<line x1="{L + pw + 12}" y1="{ly - 4}" x2="{L + pw + 34}" y2="{ly - 4}" stroke="{s["color"]}" stroke-width="2"{dash}/>')
            out.append(f'<text x="{L + pw + 40}" y="{ly}">{html.escape(s["label"])}</text>')
        out.append("</svg>")
        return "\n".join(out)

    def save(self, path) -> Path:
        path = Path(path)
        path.write_text(self.svg())
        return path


# ---- figures ---------------------------------------------------------------------------------------------------------
def fig_curves(exp_dirs: Sequence[str], out, key="val/loss", x="tokens") -> Path:
    """Loss curves of several runs on shared axes (reference: visualization/bighead_loss_curves.py)."""
    from .logging.metrics import read_metrics, series

    ch = LineChart(f"{key} against {x}", x, key, logx=True, logy=False)
    for d in exp_dirs:
        xs, ys = series(read_metrics(Path(d)), key, x=x)
        ch.add(xs, ys, Path(d).name[:40])
    return ch.save(out)


def fig_compute(runs: Sequence[str], out, key="val/loss") -> Path:
    """Loss against training compute in PFLOP-hours; `runs` are "<exp_dir>:<non-embedding parameters>" (reference:
    visualization/compute_saved.py, compare_scaling_rules.py)."""
    from .analysis import loss_vs_compute
    from .logging.metrics import read_metrics

    ch = LineChart(f"{key} against compute", "compute (PFLOP-hours)", key, logx=True, logy=True)
    for r in runs:
        d, n = r.rsplit(":", 1)
        c, l = loss_vs_compute(read_metrics(Path(d)), float(n), key)
        ch.add(c, l, Path(d).name[:40])
    return ch.save(out)


def fig_lr_law(P: Sequence[float], lr: Sequence[float], out, label="best lr") -> Path:
    """Best learning rate of every model size with the fitted law lr = a (b + P)^d (reference:
    visualization/bighead_lr_scaling.py, whose fit produced config/scaling_rules.yaml)."""
    from .analysis import fit_lr_power_law

    a, b, d, _ = fit_lr_power_law(list(P), list(lr))
    grid = np.geomspace(min(P) / 2, max(P) * 2, 100)
    ch = LineChart(f"lr = {a:.3g} ({b:.3g} + P)^{d:.3f}", "non-embedding parameters P", "peak learning rate", True, True)
    ch.add(P, lr, label, markers=True)
    ch.add(grid, a * (b + grid) ** d, "fit", dashed=True)
    return ch.save(out)


def fig_hummingbird(data: dict, out) -> Path:
    """Population risk against step for every kappa of a sweep, Adam dashed (reference: jax/hummingbird_plot.py)."""
    ch = LineChart(f"{data['args'].get('optimizer', '')}: risk against step for every kappa", "step", "population risk",
                   logx=True, logy=True)
    for name, run in data["runs"].items():
        ch.add(run["timestamps"], run["losses"], name.replace("_kappa", " k="), dashed=name == "adam")
    return ch.save(out)


def fig_hummingbird_multi(datasets: Sequence[dict], out, kappa_min: float = 0.0, color_by_clipsnr: bool = False) -> Path:
    """Several kappa sweeps (one per optimizer, each the output of `theory.generate hummingbird`) on one pair of axes:
    one colour per optimizer (or per clip-SNR), lines faint and thin at kappa_min and opaque and thick at kappa = 1,
    the Adam baseline once, dashed (reference: visualization/hummingbird_plot_from_data_multiopt.py:107-300)."""
    from .studies import palette

    ch = LineChart("risk against step: kappa sweeps of several optimizers", "step", "population risk", logx=True, logy=True)
    adam_done = False
    for data in datasets:
        opt = data["args"].get("optimizer", "")
        clip = 16.0 if opt == "adana" else float(data["args"].get("clipsnr", 1.0))
        col = palette.clipsnr_color(clip) if color_by_clipsnr else palette.color(opt, "#333333")
        first = True
        for name, run in sorted(data["runs"].items()):
            if name == "adam":
                if not adam_done:
                    ch.add(run["timestamps"], run["losses"], "Adam", "#000000", dashed=True, width=2.5)
                    adam_done = True
                continue
            kappa = float(name.rsplit("kappa", 1)[1])
            if kappa < kappa_min:
                continue
            opacity, width = palette.line_emphasis(kappa, kappa_min)
            ch.add(run["timestamps"], run["losses"], palette.display_name(opt) if first else "", col, opacity=opacity, width=width)
            first = False
    return ch.save(out)


def fig_taustats(data: dict, out, raw: bool = False) -> Path:
    """Distribution of tau at the recorded times as a dual-tail CDF: tau (regularised as the optimizer regularises it,
    unless `raw`) on a log axis against the cumulative probability on a logit axis with compressed tails, one line per
    time (reference: jax/taustats_plot_from_data.py:68-420, visualization/plot_tau_summary.py)."""
    from .studies.tau_cdf import PROB_TICKS, cdf_from_order_stats, prob_axis, regularize_tau

    n = int(data["args"]["d"]) * int(data["args"]["m"])
    ticks = [(float(prob_axis(p)[0]), f"{100 * p:g}%") for p in PROB_TICKS]
    ch = LineChart("tau: cumulative distribution over training", "tau" if raw else "regularised tau", "cumulative probability",
                   logx=True, yticks=ticks)
    for snap in data["tau"][-8:]:
        tau, prob = cdf_from_order_stats(snap["smallest"], snap["largest"], n)
        if not raw:
            tau = regularize_tau(tau, snap["step"])
        ch.add(tau, prob_axis(prob), f"step {snap['step']}")
    return ch.save(out)


def main(argv=None):
    p = argparse.ArgumentParser(prog="python -m adana_b200.figures")
    sub = p.add_subparsers(dest="cmd", required=True)
    for name in ("curves", "compute", "lr-law", "hummingbird", "hummingbird-multi", "taustats"):
        s = sub.add_parser(name)
        s.add_argument("inputs", nargs="+")
        s.add_argument("--out", required=True)
        s.add_argument("--key", default="val/loss")
    a = p.parse_args(argv)
    if a.cmd == "curves":
        return fig_curves(a.inputs, a.out, a.key)
    if a.cmd == "compute":
        return fig_compute(a.inputs, a.out, a.key)
    if a.cmd == "hummingbird-multi":
        return fig_hummingbird_multi([json.loads(Path(f).read_text()) for f in a.inputs], a.out)
    data = json.loads(Path(a.inputs[0]).read_text())
    if a.cmd == "lr-law":
        return fig_lr_law(data["P"], data["lr"], a.out)
    if a.cmd == "hummingbird":
        return fig_hummingbird(data, a.out)
    return fig_taustats(data, a.out)


if __name__ == "__main__":
    print(main())
