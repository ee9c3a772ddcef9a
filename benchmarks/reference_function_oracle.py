#!/usr/bin/env python
"""Golden values for `tests/test_studies.py`: evaluates the pure functions of the reference's figure scripts on fixed
inputs and writes the results to `tests/golden/studies_reference_values.json`.

    python benchmarks/reference_function_oracle.py --ref_root <checkout of the reference> [--out FILE]

The figure scripts import matplotlib, wandb and jax at module level and parse `sys.argv` on import, so they cannot be
imported here; instead the named function definitions are cut out of each file with `ast` and compiled into a namespace
that holds numpy, pandas and the standard modules they use.  Only functions that need nothing else are taken (the fits
that run Adagrad through jax are tested against synthetic data with known parameters instead).
"""
import argparse
import ast
import json
import math
import re
from collections import defaultdict
from pathlib import Path

import numpy as np
import pandas as pd

ROOT = Path(__file__).resolve().parent.parent


def cut(path: Path, names, extra=None):
    tree = ast.parse(path.read_text())
    keep = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    missing = set(names) - {n.name for n in keep}
    if missing:
        raise SystemExit(f"{path.name}: no function {sorted(missing)}")
    ns = {"np": np, "pd": pd, "json": json, "re": re, "math": math, "defaultdict": defaultdict,
          "Dict": dict, "List": list, "Tuple": tuple, "Optional": object, "Any": object, "print": lambda *a, **k: None}
    ns.update(extra or {})
    for fn in keep:
        fn.returns = None
        for a in fn.args.args + fn.args.kwonlyargs:
            a.annotation = None
    exec(compile(ast.Module(keep, []), str(path), "exec"), ns)
    return ns


def plain(o):
    if isinstance(o, dict):
        return {str(k): plain(v) for k, v in o.items()}
    if isinstance(o, (list, tuple)):
        return [plain(v) for v in o]
    if isinstance(o, np.ndarray):
        return [plain(v) for v in o.tolist()]
    if isinstance(o, (np.floating, float)):
        f = float(o)
        return None if math.isnan(f) else ("inf" if math.isinf(f) else f)
    if isinstance(o, (np.integer,)):
        return int(o)
    return o


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref_root", required=True)
    ap.add_argument("--out", default=str(ROOT / "tests" / "golden" / "studies_reference_values.json"))
    a = ap.parse_args()
    viz = Path(a.ref_root) / "visualization"
    G = {}

    # ---- model sizes and compute ------------------------------------------------------------------------------------
    ns = cut(viz / "compare_scaling_rules_ep.py", ["compute_params"])
    cases = [("BigHead", 6), ("BigHead", 10), ("EggHead", 5), ("EggHead", 8), ("Enoki", 8), ("Enoki_Scaled", 36),
             ("Enoki_512", 14), ("Eryngii", 9), ("Eryngii_Scaled", 16), ("Qwen3_Scaled", 6), ("Qwen3_Hoyer", 12)]
    G["compute_params"] = [{"rule": r, "size": s, "formula": f, "out": plain(ns["compute_params"](s, r, f, 2048))}
                           for r, s in cases for f in ("default", "6N1", "6N2", "M")]
    ns = cut(viz / "gamma3_factor_scaling.py", ["calculate_chinchilla_iterations", "power_law", "linear_func", "exponential_func",
                                                 "fit_function", "fit_kappa_to_gamma_formula", "fit_kappa_only_to_gamma_formula"])
    G["chinchilla_iterations"] = {str(h): ns["calculate_chinchilla_iterations"](h, "Enoki_Scaled") for h in (6, 8, 12, 24, 36)}

    # ---- gamma3 fits ---------------------------------------------------------------------------------------------------
    rng = np.random.default_rng(0)
    T = np.array([500, 1000, 2000, 4000, 8000, 16000, 500, 1000, 2000], dtype=float)
    g = 3.0 * T ** -0.45 * np.exp(rng.normal(0, 0.05, len(T)))
    w = np.array([3, 2, 1, 3, 2, 1, 5, 4, 3], dtype=float)
    G["gamma3"] = {"T": T.tolist(), "g": g.tolist(), "w": w.tolist(),
                   "power": plain(ns["fit_function"](T, g, "power", w)[0]),
                   "linear": plain(ns["fit_function"](T, g, "linear", w)[0]),
                   "exponential": plain(ns["fit_function"](T, g, "exponential", w)[0]),
                   "delta_kappa": plain(ns["fit_kappa_to_gamma_formula"](T, g, w)),
                   "kappa_only": plain(ns["fit_kappa_only_to_gamma_formula"](T, g, w)),
                   "kappa_only_negative": plain(ns["fit_kappa_only_to_gamma_formula"](T, g, w, negative=True))}

    # ---- curvature -----------------------------------------------------------------------------------------------------
    ns = cut(viz / "lr_curvature_analysis.py", ["fit_local_curvature", "compute_average_curvature", "fit_curvature_scaling_law",
                                                 "predict_loss_increase"])
    lrs = np.array([1e-4, 2e-4, 4e-4, 8e-4, 1.6e-3, 3.2e-3])
    convex = 3.2 + 0.04 * (np.log(lrs) - math.log(6e-4)) ** 2 + np.array([0.002, -0.001, 0.0005, 0.001, -0.002, 0.001])
    bumpy = np.array([3.30, 3.40, 3.25, 3.21, 3.24, 3.10])      # the parabola over all six points opens downwards
    G["curvature"] = {"lrs": lrs.tolist(), "convex": convex.tolist(), "bumpy": bumpy.tolist(),
                      "fit_convex": plain(ns["fit_local_curvature"](lrs, convex)),
                      "fit_bumpy": plain(ns["fit_local_curvature"](lrs, bumpy)),
                      "average": plain(ns["compute_average_curvature"](np.array([0.03, np.nan, 0.05, 0.04]))),
                      "power_law": plain(ns["fit_curvature_scaling_law"](np.array([1e7, 1e8, 1e9, 3e9]), np.array([0.05, 0.04, np.nan, 0.025]))),
                      "increase": plain(ns["predict_loss_increase"](2.5e9, 0.2, 0.3, -0.1))}

    # ---- compute saved and its sensitivity ---------------------------------------------------------------------------------
    ns = cut(viz / "compute_saved_sensitivity.py", ["loss_scaling_law", "compute_from_loss", "compute_saved", "compute_saved_fraction",
                                                     "loss_increase_from_lr_error", "lr_error_from_ci", "compute_saved_with_uncertainty",
                                                     "propagate_lr_to_loss_uncertainty"])
    abc = (2.5, 0.5, 0.12)
    boot = {"lr_predictions": {"1000000000": {"lr_mean": 1e-3, "lr_ci_lower": 8e-4, "lr_ci_upper": 1.3e-3},
                               "3000000000": {"lr_mean": 7e-4, "lr_ci_lower": 5e-4, "lr_ci_upper": 9e-4}}}
    curv = {"curvature_scaling_law": {"kappa_0": 0.3, "alpha": -0.1}}
    G["sensitivity"] = {"abc": abc, "bootstrap": boot, "curvature": curv,
                        "loss_at_10": ns["loss_scaling_law"](10.0, *abc), "compute_for_2.9": ns["compute_from_loss"](2.9, *abc),
                        "compute_for_floor": plain(ns["compute_from_loss"](2.5, *abc)),
                        "saved": ns["compute_saved"](2.95, 2.9, *abc), "fraction": ns["compute_saved_fraction"](2.95, 2.9, *abc),
                        "increase": ns["loss_increase_from_lr_error"](0.2, 0.04), "lr_error": ns["lr_error_from_ci"](1e-3, 8e-4, 1.3e-3),
                        "interval": plain(ns["compute_saved_with_uncertainty"](2.95, 2.9, 0.01, *abc, confidence_level=0.95)),
                        "propagate": plain(ns["propagate_lr_to_loss_uncertainty"](boot, curv, 2.6e9))}
    ns = cut(viz / "compute_saved.py", ["compute_compute_saved", "fit_lines_ols"])
    base = {8: {"final_loss": 3.5, "final_compute": 1.0, "model_compute": 1.0, "non_emb": 1e7},
            12: {"final_loss": 3.2, "final_compute": 4.0, "model_compute": 4.0, "non_emb": 5e7},
            16: {"final_loss": 3.0, "final_compute": 9.0, "model_compute": 9.0, "non_emb": 1e8}}
    cand = {8: [{"history": [(0.2, 4.0), (0.6, 3.5), (1.0, 3.4)], "final_compute": 1.0, "run_name": "a"},
                {"history": [(0.2, 3.9), (0.5, 3.45), (1.0, 3.42)], "final_compute": 1.0, "run_name": "b"}],
            12: [{"history": [(1.0, 3.6), (3.0, 3.3), (4.0, 3.25)], "final_compute": 4.0, "run_name": "c"}],
            16: [{"history": [(2.0, 3.3), (7.0, 2.99), (9.0, 2.95)], "final_compute": 9.0, "run_name": "d"}]}
    ds = [{"name": "opt", "x": [0.5, 1.0, 4.0, 9.0, 20.0, 40.0], "y": [0.1, 0.4, 1.5, 2.0, 6.0, 11.0], "weights": [1] * 6}]
    G["savings"] = {"baselines": plain(base), "candidates": plain(cand), "per_size": plain(ns["compute_compute_saved"](base, cand)),
                    "datasets": ds, "lines": plain(ns["fit_lines_ols"](ds, (1.0, 30.0)))}

    # ---- learning-rate law: selection and intervals ------------------------------------------------------------------------
    ns = cut(viz / "bighead_lr_scaling.py", ["deduplicate_lrs", "get_top_k_lrs_for_omega", "compute_confidence_intervals",
                                              "compute_lr_confidence_band"])
    rows = [{"lr": 1e-3, "val_loss": 3.30, "omega": 4.0}, {"lr": 1.02e-3, "val_loss": 3.28, "omega": 4.02}, {"lr": 2e-3, "val_loss": 3.25, "omega": 3.95},
            {"lr": 4e-3, "val_loss": 3.27, "omega": 4.0}, {"lr": 8e-3, "val_loss": 3.40, "omega": 4.05}, {"lr": 5e-4, "val_loss": 3.45, "omega": 4.0},
            {"lr": 2.5e-4, "val_loss": 3.60, "omega": 4.0}, {"lr": 1.6e-2, "val_loss": 3.9, "omega": 8.0}]
    top, rest = ns["get_top_k_lrs_for_omega"](pd.DataFrame(rows), 4.0, top_k=3, omega_tolerance=0.1, lr_tolerance=0.05)
    s = np.random.default_rng(1)
    a_s, b_s, d_s = 10 * np.exp(s.normal(0, 0.1, 50)), 3e4 * np.exp(s.normal(0, 0.2, 50)), -0.5 + s.normal(0, 0.02, 50)
    a_s[3] = np.nan
    G["lr_law"] = {"rows": rows, "top": plain(top), "rest": plain(rest),
                   "dedupe": plain(ns["deduplicate_lrs"](pd.DataFrame(rows), 0.05).to_dict("records")),
                   "a": plain(a_s), "b": plain(b_s), "d": plain(d_s),
                   "intervals": plain(ns["compute_confidence_intervals"](a_s, b_s, d_s, 0.95, [1e8, 2.5e9])),
                   "band": plain(ns["compute_lr_confidence_band"](np.array([1e7, 1e8, 1e9]), a_s, b_s, d_s, 0.9))}

    # ---- tau CDFs -----------------------------------------------------------------------------------------------------------
    ns = cut(viz / "plot_aggregated_tensors.py", ["regularize_tau", "transform_prob_to_yaxis", "reconstruct_single_cdf", "merge_cdfs",
                                                   "normalize_param_name"])
    probs = [0.0, 1e-4, 5e-4, 0.001, 0.01, 0.3, 0.5, 0.9, 0.999, 0.9995, 1.0]
    n = 5000
    tau = np.sort(np.random.default_rng(2).beta(0.5, 3.0, n))
    kmax = int(np.ceil(np.log(n) / np.log(1.1)))
    idx = np.minimum(np.unique(np.int32(1.1 ** np.arange(kmax + 1)) - 1), n - 1)
    smallest, largest = tau[idx], tau[(n - 1) - idx]
    t1, c1 = ns["reconstruct_single_cdf"](smallest, largest, n)
    t2, c2 = ns["reconstruct_single_cdf"](smallest[:20] * 1.5, largest[:25] * 0.8, 700)
    names = ["module.transformer.h.3.mlp.gate_proj.weight", "module.transformer.h.15.attn.k_norm.weight", "module.transformer.wte.weight",
             "module.lm_head.weight", "transformer.h.0.attn.c_attn.weight"]
    G["tau"] = {"probs": probs, "axis": plain(ns["transform_prob_to_yaxis"](np.array(probs))),
                "reg": plain(ns["regularize_tau"](np.array([1e-6, 0.01, 0.3, 0.5, 0.9]), 1000)),
                "n": n, "smallest": plain(smallest), "largest": plain(largest), "cdf_tau": plain(t1), "cdf_prob": plain(c1),
                "second": {"smallest": plain(smallest[:20] * 1.5), "largest": plain(largest[:25] * 0.8), "n": 700, "tau": plain(t2), "prob": plain(c2)},
                "merged": plain(ns["merge_cdfs"]([(t1, c1), (t2, c2)])),
                "names": names, "kinds": [ns["normalize_param_name"](x) for x in names]}

    # ---- colours and labels ---------------------------------------------------------------------------------------------------
    src = ast.parse((viz / "opt_colors.py").read_text())
    tables = {}
    for node in src.body:
        if isinstance(node, ast.Assign) and isinstance(node.targets[0], ast.Name) and node.targets[0].id in ("OPT_COLORS", "OPT_LINESTYLES", "OPT_DISPLAY_NAMES"):
            tables[node.targets[0].id] = ast.literal_eval(node.value)
    ns = cut(viz / "llm_hummingbird_plot.py", ["hex_to_rgb", "interpolate_color", "get_clipsnr_color"], {"OPT_COLORS": tables["OPT_COLORS"]})
    clips = [0.1, 0.25, 0.5, 1.0, 2.0, 8.0, 100.0, 1000.0]
    G["palette"] = {**tables, "clipsnr": clips, "clipsnr_colors": [plain(ns["get_clipsnr_color"](c)) for c in clips]}
    ns = cut(viz / "hoyer_final_loss.py", ["get_hoyer_linestyle", "get_hoyer_label"], {"HOYER_LINESTYLES": {}})
    coeffs = [0, 1e-6, 1e-4, 3e-4, 1e-3, 2.5e-3, 1e-2]
    G["hoyer"] = {"coeffs": coeffs, "linestyles": [ns["get_hoyer_linestyle"](c) for c in coeffs], "labels": [ns["get_hoyer_label"](c) for c in coeffs]}
    ns = cut(viz / "llm_hummingbird_slice_plot.py", ["is_reliable_kappa"])
    ks = [0.0, 0.05, 0.1, 0.15, 0.5, 0.75, 0.8, 0.85, 1.0]
    G["tenths"] = {"kappas": ks, "keep": [bool(ns["is_reliable_kappa"](k)) for k in ks]}

    Path(a.out).write_text(json.dumps(G, indent=0))
    print(f"wrote {a.out}: {sorted(G)}")


if __name__ == "__main__":
    main()
