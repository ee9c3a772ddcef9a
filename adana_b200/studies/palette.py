"""One colour, line style and legend name per optimizer, so every figure of the studies shows the same optimizer the
same way; plus the continuous scales (kappa, clip-SNR, Hoyer coefficient) the sweep figures colour their lines by.

Counterpart of the reference's visualization/opt_colors.py (names and hex colours are kept so figures made here and
there can sit side by side) and of the colour helpers its figure scripts repeat (llm_hummingbird_plot.py:50-89,
hoyer_loss_curves.py:303-328, hoyer_final_loss.py:34-64).  No plotting package is needed: the two colour maps are
piecewise-linear through eight or nine anchor colours.
"""
from __future__ import annotations

import math
from typing import Sequence, Tuple

_FAMILY = {
    "adamw": ("#1f77b4", "AdamW"),
    "adamw-decaying-wd": ("#00CED1", "AdamW (DW)"),
    "mk4": ("#d62728", "DANA-Star-MK4"),
    "dana": ("#2ca02c", "DANA"),
    "dana-mk4": ("#8c564b", "DANA-MK4"),
    "dana-mk4-kappa-0-75": ("#A0522D", "DANA-MK4 κ=0.75"),
    "dana-mk4-kappa-0-85": ("#CD853F", "DANA-MK4 κ=0.85"),
    "dana-star": ("#7f7f7f", "DANA-Star"),
    "dana-star-mk4": ("#d62728", "DANA-Star-MK4"),
    "dana-star-mk4-kappa-0-75": ("#DC143C", "DANA-Star-MK4 κ=0.75"),
    "dana-star-mk4-kappa-0-85": ("#FF6347", "DANA-Star-MK4 κ=0.85"),
    "adana": ("#bcbd22", "ADANA"),
    "adana-kappa-0-85": ("#228B22", "ADANA κ=0.85"),
    "dana-star-no-tau": ("#bcbd22", "ADANA"),
    "dana-star-no-tau-kappa-0-75": ("#bcbd22", "ADANA κ=0.75"),
    "dana-star-no-tau-kappa-0-8": ("#006400", "ADANA κ=0.8"),
    "dana-star-no-tau-kappa-0-85": ("#228B22", "ADANA κ=0.85"),
    "dana-star-no-tau-kappa-0-9": ("#32CD32", "ADANA κ=0.9"),
    "dana-star-no-tau-kappa-1-0": ("#00FF00", "ADANA κ=1.0"),
    "dana-star-no-tau-dana-constant": ("#FF6347", "ADANA-DanaConst"),
    "dana-star-no-tau-beta2-constant": ("#1E90FF", "ADANA-β₂Const"),
    "dana-star-no-tau-beta1": ("#FF1493", "ADANA-β₁"),
    "dana-star-no-tau-dana-constant-beta2-constant": ("#8A2BE2", "ADANA-DanaConst-β₂Const"),
    "dana-star-no-tau-dana-constant-beta1": ("#FF8C00", "ADANA-DanaConst-β₁"),
    "dana-star-no-tau-dana-constant-beta2-constant-beta1": ("#20B2AA", "ADANA-DanaConst-β₂Const-β₁"),
    "ademamix": ("#9467bd", "Ademamix"),
    "ademamix-decaying-wd": ("#e377c2", "Ademamix (DW)"),
    "d-muon": ("#ff7f0e", "Muon"),
    "muon": ("#ff7f0e", "Muon"),
    "manau": ("#8B4513", "Manau"),
    "manau-hard": ("#DC143C", "Manau-Hard"),
    "laprop": ("#17becf", "LaProp"),
    "logadam": ("#FFD700", "LogAdam"),
    "logadam-nesterov": ("#FFA500", "LogAdam-Nesterov"),
}
OPT_COLORS = {k: v[0] for k, v in _FAMILY.items()}
OPT_DISPLAY_NAMES = {k: v[1] for k, v in _FAMILY.items()}
OPT_LINESTYLES = {k: "--" for k in ("dana-mk4", "dana-star-mk4", "dana-mk4-kappa-0-85", "dana-star-mk4-kappa-0-85", "mk4")}

# evenly spaced anchors of the two perceptually uniform maps (public colour tables, rounded)
_VIRIDIS = ["#440154", "#472d7b", "#3b528b", "#2c728e", "#21918c", "#28ae80", "#5ec962", "#addc30", "#fde725"]
_PLASMA = ["#0d0887", "#5402a3", "#8b0aa5", "#b93289", "#db5c68", "#f48849", "#febc2a", "#f0f921"]


def hex_to_rgb(h: str) -> Tuple[float, float, float]:
    h = h.lstrip("#")
    return tuple(int(h[i:i + 2], 16) / 255.0 for i in (0, 2, 4))


def rgb_to_hex(rgb: Sequence[float]) -> str:
    return "#" + "".join(f"{max(0, min(255, int(round(c * 255)))):02x}" for c in rgb[:3])


def mix(c0: str, c1: str, t: float) -> str:
    """The colour a fraction t of the way from c0 to c1 (both "#rrggbb")."""
    a, b = hex_to_rgb(c0), hex_to_rgb(c1)
    return rgb_to_hex([a[i] + t * (b[i] - a[i]) for i in range(3)])


def _ramp(anchors, t: float) -> str:
    t = min(1.0, max(0.0, float(t))) * (len(anchors) - 1)
    i = min(int(t), len(anchors) - 2)
    return mix(anchors[i], anchors[i + 1], t - i)


def viridis(t: float) -> str:
    return _ramp(_VIRIDIS, t)


def plasma(t: float) -> str:
    return _ramp(_PLASMA, t)


def color(opt: str, default: str = "#000000") -> str:
    return OPT_COLORS.get(opt, default)


def display_name(opt: str) -> str:
    return OPT_DISPLAY_NAMES.get(opt, opt)


def linestyle(opt: str) -> str:
    return OPT_LINESTYLES.get(opt, "-")


def kappa_color(kappa: float, lo: float = 0.75, hi: float = 1.0) -> str:
    """Colour of a kappa-ablation line: viridis over [0.75, 1]."""
    return viridis((kappa - lo) / (hi - lo))


def kappa_label(kappa: float) -> str:
    return f"κ = {kappa:g}"


def clipsnr_color(clipsnr: float) -> str:
    """ADANA's colour for an effectively unclipped run (>= 100), MK4's red at 0.5, dark red at <= 0.25, and in
    between the mix of the two at the position of log10(clipsnr) between log10(0.5) and log10(100)."""
    if clipsnr >= 100:
        return OPT_COLORS["adana"]
    if clipsnr <= 0.25:
        return "#8B0000"
    if clipsnr <= 0.5:
        return OPT_COLORS["mk4"]
    t = (math.log10(clipsnr) - math.log10(0.5)) / (math.log10(100) - math.log10(0.5))
    return mix(OPT_COLORS["mk4"], OPT_COLORS["adana"], t)


def log_scale_color(value: float, lo: float, hi: float) -> str:
    """Plasma over the lower 80 % of its range at the position of log10(value) in [log10 lo, log10 hi]."""
    if lo == hi:
        return plasma(0.4)
    return plasma(0.8 * (math.log10(value) - math.log10(lo)) / (math.log10(hi) - math.log10(lo)))


def hoyer_linestyle(coeff: float) -> str:
    if coeff == 0 or coeff < 1e-5:
        return "-"
    if coeff < 5e-4:
        return "--"
    if coeff < 5e-3:
        return "-."
    return ":"


def hoyer_label(coeff: float) -> str:
    if coeff == 0 or coeff < 1e-6:
        return "λ=0"
    e = int(math.floor(math.log10(coeff)))
    m = coeff / 10 ** e
    return f"λ=1e{e}" if abs(m - 1.0) < 0.01 else f"λ={m:.1f}e{e}"


def line_emphasis(kappa: float, kappa_min: float) -> Tuple[float, float]:
    """(opacity, width) of a kappa-sweep line: faint and thin at kappa_min, opaque and thick at kappa = 1."""
    if kappa_min >= 1.0:
        return 1.0, 2.0
    u = (kappa - kappa_min) / (1.0 - kappa_min)
    return max(0.25, min(1.0, 0.25 + 0.75 * u)), 1.0 + 2.0 * u
