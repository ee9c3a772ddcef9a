"""Scaling studies (`adana_b200/studies`).  Where the reference's figure scripts have a pure function for a quantity,
the value is compared with `tests/golden/studies_reference_values.json`, which `benchmarks/reference_function_oracle.py`
computed by running that function (cut out of the script with `ast`) on the inputs stored in the same file.  The fits
the reference runs through jax are checked on synthetic data with known parameters; the run table, the cache and the
command line are checked end to end on experiment folders written here."""
import json
import math
import pickle
from pathlib import Path

import numpy as np
import pytest

from adana_b200.studies import curvature, gamma3, loss_laws, lr_law, palette, panels, savings, sizes, sweeps, tau_cdf
from adana_b200.studies.runs import CachedRuns, LocalRuns, Run, flatten_config, lr_sweep_table, select

G = json.loads((Path(__file__).parent / "golden" / "studies_reference_values.json").read_text())


def _f(v):
    return math.nan if v is None else (math.inf if v == "inf" else v)


# ---- sizes -------------------------------------------------------------------------------------------------------------
def test_model_sizes_and_compute_formulas_match_reference():
    for case in G["compute_params"]:
        m, ref = sizes.model_size(case["size"], case["rule"]), case["out"]
        assert (m.non_emb, m.total_params, m.n_layer, m.n_head, m.n_embd) == \
            (ref["non_emb"], ref["total_params"], ref["n_layer"], ref["n_head"], ref["n_embd"]), case
        assert m.compute_pfh(case["formula"], 2048) == pytest.approx(ref["compute"], rel=1e-12)
    for h, its in G["chinchilla_iterations"].items():
        assert sizes.model_size(int(h), "Enoki_Scaled").chinchilla_iterations() == its
    with pytest.raises(ValueError):
        sizes.model_size(8, "Shiitake")
    # the scaling engine of the launcher and the study table agree on the flagship
    from adana_b200.config.scaling import compute_dimensions

    for rule, study_rule, heads in (("enoki", "Enoki_Scaled", 36), ("qwen3", "Qwen3_Scaled", 16)):
        dims, m = compute_dimensions(rule, heads), sizes.model_size(heads, study_rule)
        assert (dims["n_layer"], dims["n_embd"]) == (m.n_layer, m.n_embd)


# ---- learning-rate law ------------------------------------------------------------------------------------------------
def test_lr_selection_matches_reference():
    g = G["lr_law"]
    assert [(r["lr"], r["val_loss"]) for r in lr_law.dedupe_lrs(g["rows"])] == [(r["lr"], r["val_loss"]) for r in g["dedupe"]]
    top, rest = lr_law.top_k_lrs(g["rows"], 3, omega=4.0, omega_tol=0.1)
    assert top == g["top"]
    assert [(r["lr"], pytest.approx(r["distance_from_optimal"])) for r in rest] == \
        [(r["lr"], r["distance_from_optimal"]) for r in g["rest"]]


def test_lr_intervals_match_reference():
    g = G["lr_law"]
    a, b, d = (np.array([_f(x) for x in g[k]]) for k in "abd")
    mine = lr_law.confidence_intervals(a, b, d, 0.95, [1e8, 2.5e9])
    ref = g["intervals"]
    assert mine["n_valid_samples"] == ref["n_valid_samples"]
    for k in "abd":
        for stat, v in ref["parameters"][k].items():
            assert mine["parameters"][k][stat] == pytest.approx(v, rel=1e-10)
    for P, d_ref in ref["lr_predictions"].items():
        for stat, v in d_ref.items():
            assert mine["lr_predictions"][P][stat] == pytest.approx(v, rel=1e-10)
    band = lr_law.confidence_band([1e7, 1e8, 1e9], a, b, d, 0.9)
    for x, y in zip(band, g["band"]):
        np.testing.assert_allclose(x, y, rtol=1e-10)


def test_weighted_lr_law_recovers_parameters_and_is_the_minimum():
    rng = np.random.default_rng(0)
    P = np.repeat(np.array([2e6, 1e7, 5e7, 2e8, 1e9, 3e9]), 3)
    w = np.tile([3.0, 2.0, 1.0], 6)
    lr = 12.0 * (4e4 + P) ** -0.52
    a, b, d, err = lr_law.fit_weighted(P, lr, w)
    assert (a, b, d) == (pytest.approx(12.0, rel=1e-3), pytest.approx(4e4, rel=1e-2), pytest.approx(-0.52, rel=1e-4))
    assert err < 1e-10
    noisy = lr * np.exp(rng.normal(0, 0.05, len(P)))
    a, b, d, err = lr_law.fit_weighted(P, noisy, w)

    def objective(a, b, d):      # the reference's loss: weights w^2 P on squared log residuals
        cw = w * w * P
        return float(np.sum(cw * (np.log(noisy) - np.log(a * (b + P) ** d)) ** 2) / np.sum(cw))

    assert objective(a, b, d) == pytest.approx(err, rel=1e-9)
    for da, db, dd in [(1.05, 1, 0), (1, 1.3, 0), (1, 1, 0.01), (0.97, 0.8, -0.005)]:
        assert objective(a * da, b * db, d + dd) >= err
    with pytest.raises(ValueError):
        lr_law.fit_weighted([1e7, 1e7], [1e-3, 1.1e-3])


def test_lr_law_study_with_bootstrap():
    rng = np.random.default_rng(1)
    table = {}
    for h in (8, 12, 16, 24, 32):
        P = sizes.model_size(h, "Enoki_Scaled").non_emb
        best = 15.0 * (3e4 + P) ** -0.5
        table[h] = [{"lr": best * f, "val_loss": 3.0 + 0.05 * math.log(f) ** 2 + rng.normal(0, 1e-4), "omega": 4.0}
                    for f in (0.25, 0.5, 0.7, 1.0, 1.4, 2.0, 4.0)]
    rep = lr_law.study(table, "Enoki_Scaled", k=3, omega=4.0, n_boot=40, extrapolate_sizes=[36, 48])
    assert rep["fit"]["d"] == pytest.approx(-0.5, abs=0.05)
    P36 = sizes.model_size(36, "Enoki_Scaled").non_emb
    pred = rep["bootstrap"]["lr_predictions"][str(P36)]
    assert pred["lr_ci_lower"] <= pred["lr_median"] <= pred["lr_ci_upper"]
    assert pred["lr_median"] == pytest.approx(15.0 * (3e4 + P36) ** -0.5, rel=0.15)
    assert all(len(v["top_k_data"]) == 3 for v in rep["sizes"].values())


# ---- curvature -------------------------------------------------------------------------------------------------------
def test_curvature_matches_reference():
    g = G["curvature"]
    np.testing.assert_allclose(curvature.fit_parabola(g["lrs"], g["convex"]), g["fit_convex"], rtol=1e-9)
    np.testing.assert_allclose(curvature.fit_parabola(g["lrs"], g["bumpy"]), [_f(x) for x in g["fit_bumpy"]], rtol=1e-9)
    assert curvature.mean_curvature([0.03, math.nan, 0.05, 0.04]) == pytest.approx(tuple(g["average"]))
    assert curvature.curvature_power_law([1e7, 1e8, 1e9, 3e9], [0.05, 0.04, math.nan, 0.025]) == pytest.approx(tuple(g["power_law"]))
    assert curvature.loss_increase_at(2.5e9, 0.2, 0.3, -0.1) == pytest.approx(g["increase"])
    assert all(math.isnan(x) for x in curvature.fit_parabola([1e-3, 2e-3, 4e-3], [3.0, 3.2, 3.1]))


def test_curvature_study_report_feeds_the_sensitivity():
    table = {h: [{"lr": 1e-3 * f, "val_loss": 3.0 - 0.01 * h + 0.04 * math.log(f) ** 2, "omega": 4.0} for f in (0.25, 0.5, 1, 2, 4)]
             for h in (8, 12, 16)}
    rep = curvature.study(table, "Enoki_Scaled", extrapolation_sizes=[24, 36])
    assert rep["average_curvature"]["mean"] == pytest.approx(0.04, rel=1e-6)
    assert all(v["lr_star"] == pytest.approx(1e-3, rel=1e-6) for v in rep["per_size"].values())
    assert rep["curvature_scaling_law"]["alpha"] == pytest.approx(0.0, abs=1e-6)
    assert rep["loss_sensitivity"]["delta_loss"]["36"]["0.2"]["mean_kappa"] == pytest.approx(0.04 * math.log(1.2) ** 2)
    boot = {"lr_predictions": {str(sizes.model_size(36, "Enoki_Scaled").non_emb): {"lr_mean": 1e-3, "lr_ci_lower": 8e-4, "lr_ci_upper": 1.2e-3}}}
    std, err = savings.loss_spread_from_lr(boot, rep, sizes.model_size(36, "Enoki_Scaled").non_emb)
    assert err == pytest.approx(0.2) and std == pytest.approx(0.04 * math.log(1.2) ** 2, rel=1e-4)


# ---- loss laws -------------------------------------------------------------------------------------------------------
def test_single_and_broken_laws_recover_known_parameters():
    C = np.geomspace(0.01, 100, 14)
    L = loss_laws.single(C, 1.8, 0.9, 0.15)
    f = loss_laws.fit_single(C, L)
    assert (f["a"], f["b"], f["c"]) == (pytest.approx(1.8, abs=1e-3), pytest.approx(0.9, abs=1e-3), pytest.approx(0.15, abs=1e-3))
    assert f["r_squared"] > 0.999999 and np.abs(f["residuals"]).max() < 1e-4
    f0 = loss_laws.fit_single(C, loss_laws.single(C, 0.0, 3.0, 0.05), force_a_zero=True)
    assert f0["a"] == 0.0 and (f0["b"], f0["c"]) == (pytest.approx(3.0, rel=1e-4), pytest.approx(0.05, rel=1e-3))
    # a curve with two regimes: the broken law fits what the single law cannot
    Lb = loss_laws.broken(C, 1.5, 0.6, 0.4, 1.2, 0.05)
    fb, fs = loss_laws.fit_broken(C, Lb), loss_laws.fit_single(C, Lb)
    assert np.abs(fb["residuals"]).max() < 2e-3 < np.abs(fs["residuals"]).max()
    fa = loss_laws.fit_broken(C, Lb, a=1.5)
    assert fa["a"] == 1.5 and np.abs(fa["residuals"]).max() < 1e-3


def test_joint_fit_shares_the_floor_and_multiplier_is_consistent():
    C = np.geomspace(0.05, 60, 10)
    base = loss_laws.broken(C, 1.7, 0.5, 0.30, 1.0, 0.06)
    fast = loss_laws.broken(C * 1.5, 1.7, 0.5, 0.30, 1.0, 0.06)      # the same law reached with 1.5x less compute
    fit = loss_laws.fit_joint([{"name": "adamw", "compute": C, "loss": base}, {"name": "dana-star-mk4", "compute": C, "loss": fast}], "broken")
    assert set(fit["curves"]) == {"adamw", "dana-star-mk4"} and 0.0 < fit["a"] < 0.99 * fast.min()
    assert min(c["r_squared"] for c in fit["curves"].values()) > 0.9999
    x, gpw = loss_laws.multiplier_piecewise(C, fast, C, base)
    np.testing.assert_allclose(gpw[1:-1], 1.5, rtol=0.02)            # interpolation inside the baseline's range
    assert gpw[-1] == pytest.approx(1.5, rel=0.05)                   # extrapolated beyond its best loss
    xs, gfit = loss_laws.multiplier_from_fits(C, fit["a"], fit["curves"]["dana-star-mk4"], fit["curves"]["adamw"])
    np.testing.assert_allclose(gfit, 1.5, rtol=0.05)
    single = loss_laws.fit_joint([{"name": "a", "compute": C, "loss": loss_laws.single(C, 1.2, 0.8, 0.2)},
                                  {"name": "b", "compute": C, "loss": loss_laws.single(C, 1.2, 0.6, 0.25)}], "single", compute_weight=True)
    assert single["a"] == pytest.approx(1.2, abs=0.02) and single["curves"]["b"]["c"] == pytest.approx(0.25, abs=0.02)
    assert loss_laws.baseline_compute_for_loss(float(base[3]), C, base) == pytest.approx(C[3])


# ---- savings ---------------------------------------------------------------------------------------------------------
def test_compute_saved_and_sensitivity_match_reference():
    g = G["savings"]
    base = {int(k): v for k, v in g["baselines"].items()}
    cand = {int(k): [{**r, "history": [tuple(h) for h in r["history"]]} for r in v] for k, v in g["candidates"].items()}
    assert savings.saved_per_size(base, cand) == [{**r, "size": int(r["size"])} for r in g["per_size"]]
    mine = savings.fit_savings_lines(g["datasets"], (1.0, 30.0))["curves"]["opt"]
    for k in ("b", "c", "r_squared", "n_points"):
        assert mine[k] == pytest.approx(g["lines"]["curves"]["opt"][k])
    s = G["sensitivity"]
    abc = s["abc"]
    assert savings.loss_at(10.0, *abc) == pytest.approx(s["loss_at_10"])
    assert savings.compute_for(2.9, *abc) == pytest.approx(s["compute_for_2.9"])
    assert savings.compute_for(2.5, *abc) == math.inf and s["compute_for_floor"] == "inf"
    assert savings.saved(2.95, 2.9, *abc) == pytest.approx(s["saved"])
    assert savings.saved_fraction(2.95, 2.9, *abc) == pytest.approx(s["fraction"])
    assert curvature.loss_increase(0.2, 0.04) == pytest.approx(s["increase"])
    assert savings.lr_error_from_interval(1e-3, 8e-4, 1.3e-3) == pytest.approx(s["lr_error"])
    iv = savings.saved_fraction_interval(2.95, 2.9, 0.01, *abc, level=0.95)
    for k, v in s["interval"].items():
        assert iv[k] == pytest.approx(v, rel=1e-9)
    assert savings.loss_spread_from_lr(s["bootstrap"], s["curvature"], 2.6e9) == pytest.approx(tuple(s["propagate"]))
    rep = savings.sensitivity({"adamw": s["bootstrap"], "dana-mk4": s["bootstrap"]}, s["curvature"], {"adamw": 2.95, "dana-mk4": 2.9},
                              "adamw", 2.6e9, *abc)
    row = next(r for r in rep["analysis"] if r["optimizer"] == "dana-mk4")
    cs = row["compute_saved"]      # a lower loss costs the law more compute: the fraction is negative, its size is the gain
    assert min(cs["ci_lower"], cs["ci_upper"]) < cs["mean"] < max(cs["ci_lower"], cs["ci_upper"]) < 0


# ---- gamma3 ----------------------------------------------------------------------------------------------------------
def test_gamma3_fits_match_reference_and_ranking():
    g = G["gamma3"]
    T, y, w = g["T"], g["g"], g["w"]
    for kind in ("power", "linear", "exponential"):
        assert gamma3.fit(T, y, kind, w) == pytest.approx(tuple(g[kind]), rel=1e-9)
    (dk, per_point), ref = gamma3.fit_delta_kappa(T, y, w), g["delta_kappa"]
    assert dk == pytest.approx(tuple(ref[0]), rel=1e-9)
    np.testing.assert_allclose(per_point, ref[1], rtol=1e-12)
    assert gamma3.fit_kappa_only(T, y, w) == pytest.approx(g["kappa_only"])
    assert gamma3.fit_kappa_only(T, y, w, negative=True) == pytest.approx(g["kappa_only_negative"])
    assert gamma3.fit([1.0], [1.0]) is None
    rows = [{"size": 8, "iterations": 1000, "gamma_3_factor": gf, "val_loss": 3.0 + abs(math.log(gf / 0.2))} for gf in (0.05, 0.1, 0.2, 0.4, 0.8)]
    rows += [{"size": 8, "iterations": 2000, "gamma_3_factor": 0.1, "val_loss": 2.9}, {"size": 8, "iterations": 2000, "gamma_3_factor": 0.2, "val_loss": 2.95}]
    pts = gamma3.ranked_points(rows, top_k=3)
    assert [(p["gamma_3_factor"], p["weight"]) for p in pts] == [(0.2, 5), (0.1, 4), (0.4, 4)] or \
        [(p["gamma_3_factor"], p["weight"]) for p in pts][0] == (0.2, 5)          # the group of two runs is dropped
    assert all(p["iterations"] == 1000 for p in pts)
    chin = sizes.model_size(8, "Enoki_Scaled").chinchilla_iterations()
    kept = gamma3.within_chinchilla_window([{"size": 8, "iterations": chin // 4}, {"size": 8, "iterations": chin * 3}], "Enoki_Scaled", 0.1, 2.0)
    assert [r["iterations"] for r in kept] == [chin // 4]
    rep = gamma3.study([{"size": 8, "iterations": t, "gamma_3_factor": 2.0 * t ** -0.4 * f, "val_loss": 3.0 + abs(math.log(f))}
                        for t in (500, 1000, 2000, 4000) for f in (0.5, 1.0, 2.0)], top_k=1)
    assert rep["params"] == pytest.approx((2.0, -0.4), rel=1e-6)


# ---- tau distributions ---------------------------------------------------------------------------------------------
def test_tau_cdf_pieces_match_reference():
    g = G["tau"]
    np.testing.assert_allclose(tau_cdf.prob_axis(g["probs"]), g["axis"], rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(tau_cdf.regularize_tau([1e-6, 0.01, 0.3, 0.5, 0.9], 1000), g["reg"], rtol=1e-12)
    t, c = tau_cdf.cdf_from_order_stats(g["smallest"], g["largest"], g["n"])
    np.testing.assert_allclose(t, g["cdf_tau"], rtol=1e-12)
    np.testing.assert_allclose(np.sort(c), np.sort(g["cdf_prob"]), rtol=1e-12)
    s = g["second"]
    t2, c2 = tau_cdf.cdf_from_order_stats(s["smallest"], s["largest"], s["n"])
    np.testing.assert_allclose(t2, s["tau"], rtol=1e-12)
    m = tau_cdf.merge_cdfs([(np.array(g["cdf_tau"]), np.array(g["cdf_prob"])), (np.array(s["tau"]), np.array(s["prob"]))])
    np.testing.assert_allclose(m["tau_values"], g["merged"]["tau_values"], rtol=1e-12)
    np.testing.assert_allclose(m["cdf_values"], g["merged"]["cdf_values"], rtol=1e-12)
    assert [tau_cdf.kind_of(n) for n in g["names"]] == g["kinds"]
    assert tau_cdf.cdf_from_order_stats([], [], 10)[0].size == 0


def test_tau_summary_reads_what_the_collector_writes(tmp_path):
    import torch
    from types import SimpleNamespace

    from adana_b200.logging.tau_stats import TauStatsCollector

    names = ["module.transformer.wte.weight", "module.transformer.h.0.attn.c_attn.weight", "module.transformer.h.1.attn.c_attn.weight",
             "module.transformer.h.0.mlp.c_fc.weight", "module.transformer.h.1.mlp.c_fc.weight", "module.lm_head.weight"]
    params = [torch.nn.Parameter(torch.zeros(64, 32)) for _ in names]
    opt = SimpleNamespace(param_groups=[{"params": params, "param_names": names}], state={})
    cfg = SimpleNamespace(iterations=1000, eval_interval=1, model="enoki", n_head=4, opt="dana-star-mk4", kappa=0.85)
    col = TauStatsCollector(tmp_path, cfg, names)
    gen = torch.Generator().manual_seed(0)
    for it in (10, 20, 40, 80, 160):
        for p in params:
            opt.state[p] = {"tau": torch.rand(p.shape, generator=gen) ** (1 + it / 40)}
        col.eval_step_counter = it
        col.collect(opt, it)
    rep = tau_cdf.summary(tmp_path / "tau_stats")
    assert set(rep["groups"]) == {"Embedding", "Attention", "MLP", "Output"} and rep["iterations"] == [10, 20, 80, 160]
    assert rep["groups"]["Attention"]["tensors"] == 2
    line = rep["groups"]["MLP"]["lines"][-1]
    assert np.all(np.diff(line["tau"]) >= 0) and np.all(np.diff(line["prob"]) >= -1e-12) and line["prob"][-1] == pytest.approx(1.0)
    raw = tau_cdf.summary(tmp_path / "tau_stats", raw=True)["groups"]["MLP"]["lines"]
    med = [float(np.interp(0.5, l["prob"], l["tau"])) for l in raw]
    assert med[0] > med[-1]                                           # tau ** (1 + it/40) shrinks with the iteration
    exact = float(np.median(np.concatenate([opt.state[params[i]]["tau"].flatten().numpy() for i in (3, 4)])))
    assert med[-1] == pytest.approx(exact, rel=0.15)
    kinds = tau_cdf.all_kinds(tmp_path / "tau_stats", iterations=[160])
    assert "Transformer attn.c_attn.weight" in kinds["groups"] and len(kinds["groups"]) == 4
    out = panels.tau_cdf(rep["groups"]["MLP"], tmp_path / "mlp.svg", "MLP")
    assert "99.9%" in out.read_text() and out.read_text().count("<polyline") == 4


# ---- palette -----------------------------------------------------------------------------------------------------------
def test_palette_matches_reference_tables():
    g = G["palette"]
    for k, v in g["OPT_COLORS"].items():
        assert palette.color(k).lower() == v.lower(), k
    for k, v in g["OPT_DISPLAY_NAMES"].items():
        assert palette.display_name(k) == v
    assert {k for k in palette.OPT_COLORS if palette.linestyle(k) == "--"} == set(g["OPT_LINESTYLES"])
    for clip, ref in zip(g["clipsnr"], g["clipsnr_colors"]):
        mine = palette.hex_to_rgb(palette.clipsnr_color(clip))
        want = palette.hex_to_rgb(ref) if isinstance(ref, str) else tuple(ref)
        assert mine == pytest.approx(want, abs=1 / 255)
    h = G["hoyer"]
    assert [palette.hoyer_linestyle(c) for c in h["coeffs"]] == h["linestyles"]
    assert [palette.hoyer_label(c) for c in h["coeffs"]] == h["labels"]
    assert [sweeps.on_tenths_grid(k) for k in G["tenths"]["kappas"]] == G["tenths"]["keep"]
    assert palette.viridis(0.0) == "#440154" and palette.viridis(1.0) == "#fde725" and palette.plasma(0.0) == "#0d0887"
    assert palette.kappa_color(0.75) == palette.viridis(0) and palette.line_emphasis(1.0, 0.5) == (1.0, 3.0)


# ---- run table, cache, command line ---------------------------------------------------------------------------------
def _write_run(root, name, cfg, final_loss, curve):
    d = root / name
    d.mkdir(parents=True)
    (d / "summary.json").write_text(json.dumps({"args": cfg, "final-val/loss": final_loss, "iter": cfg["iterations"]}))
    with open(d / "metrics.jsonl", "w") as f:
        for it, loss in curve:
            f.write(json.dumps({"iter": it, "tokens": it * 65536, "val/loss": loss, "iter_dt": 0.5, "optimizer/auto_factor": 0.5,
                                "optimizer/kappa_factor_schedule": (1 + it) ** 0.15, "optimizer/alpha_schedule": min(2.0, 0.5 * (1 + it) ** 0.15),
                                "optimizer/m_norm": 1.0 / it}) + "\n")


@pytest.fixture()
def runs_root(tmp_path):
    root = tmp_path / "exps"
    for h in (8, 12, 16):
        P = sizes.model_size(h, "Enoki_Scaled").non_emb
        for opt, speed in (("adamw", 1.0), ("dana-star-mk4", 1.4)):
            best = 20.0 * (3e4 + P) ** -0.5
            for f in (0.5, 1.0, 2.0):
                its = 1000
                lr = best * f
                cfg = {"opt": opt, "n_head": h, "n_layer": 3 * h // 4, "lr": lr, "iterations": its, "kappa": 0.85, "clipsnr": 2.0,
                       "world_size": 2, "wandb_group": "sweep"}
                cfg.update({"weight_decay": 4.0 / 100, "wd_ts": 100} if opt != "adamw" else {"weight_decay": 4.0 / (lr * its)})
                floor = 2.0 + 3.0 * (sizes.model_size(h, "Enoki_Scaled").compute_pfh() * speed) ** -0.2 + 0.05 * math.log(f) ** 2
                curve = [(it, floor + 2.0 * (it / its) ** -0.5 - 2.0) for it in (100, 200, 400, 700, 1000)]
                _write_run(root, f"{opt}_h{h}_lr{f}", cfg, floor, curve)
    _write_run(root, "unfinished", {"opt": "adamw", "n_head": 8, "lr": 1e-3, "iterations": 5000, "weight_decay": 0.8}, 9.9, [(100, 9.9)])
    (root / "unfinished" / "summary.json").write_text(json.dumps({"args": {"opt": "adamw", "n_head": 8, "lr": 1e-3, "iterations": 5000,
                                                                           "weight_decay": 0.8}, "final-val/loss": 9.9, "iter": 100}))
    return root


def test_run_table_selection_and_cache(runs_root, tmp_path):
    src = LocalRuns(runs_root)
    runs = src.fetch()
    assert len(runs) == 19 and len(select(runs, opt="adamw")) == 9          # the unfinished run is left out
    r = next(r for r in runs if r.name == "dana-star-mk4_h8_lr1.0")
    assert r.omega() == pytest.approx(4.0) and r.omega(lr_coupled=True) == pytest.approx(4.0 * r.config["lr"])
    assert next(r for r in runs if r.name == "adamw_h12_lr2.0").omega() == pytest.approx(4.0)
    assert len(select(runs, opt="adamw", omega=4.0)) == 9 and len(select(runs, omega=1.0)) == 0
    assert len(src.fetch({"group": "sweep", "opt": "adamw"})) == 9
    assert flatten_config({"lr": {"value": 0.1, "desc": None}, "opt": "adamw"}) == {"lr": 0.1, "opt": "adamw"}
    assert flatten_config('{"a": {"value": 1}}') == {"a": 1} and flatten_config("not json") == {}
    table = lr_sweep_table(runs, "n_head", opt="dana-star-mk4", omega=4.0)
    assert sorted(table) == [8, 12, 16] and all(len(v) == 3 for v in table.values())

    cached = CachedRuns(src, tmp_path / "cache")
    first = cached.fetch({"group": "sweep"})
    hist = first[0].history()
    second = CachedRuns(LocalRuns(runs_root), tmp_path / "cache").fetch({"group": "sweep"})
    assert [r.to_json() for r in first] == [r.to_json() for r in second] and second[0].history() == hist
    moved = CachedRuns(LocalRuns(runs_root), tmp_path / "cache")
    (runs_root / first[0].name / "metrics.jsonl").unlink()                     # the history now exists only in the cache
    again = moved.fetch({"group": "sweep"})
    assert moved.hits == 1 and moved.misses == 0 and again[0].history() == hist
    fresh = CachedRuns(LocalRuns(runs_root), tmp_path / "cache", force_refresh=True)
    assert fresh.fetch({"group": "sweep"})[0].history() == [] and fresh.misses == 1


def test_sweep_studies_on_local_runs(runs_root, tmp_path):
    runs = LocalRuns(runs_root).fetch()
    best = sweeps.best_runs_per_size(runs, "Enoki_Scaled", "adamw")
    assert sorted(best) == [8, 12, 16] and all(d["run"].endswith("lr1.0") for d in best.values())
    P8 = sizes.model_size(8, "Enoki_Scaled").non_emb
    assert best[8]["compute"][-1] == pytest.approx(6.0 * P8 * 1000 * 65536 / 3600e15)
    rows = sweeps.gpu_hours_by_size(sweeps.gpu_hours_rows(runs, "Enoki_Scaled", "adamw"))
    assert [r["size"] for r in rows] == [8, 12, 16] and rows[0]["num_runs"] == 4
    assert rows[1]["gpu_hours"] == pytest.approx(0.5 * 1000 * 2 / 3600)
    text = sweeps.gpu_hours_table(rows)
    assert "Total" in text and sweeps.format_params(2.5e9) == "2.50B" and sweeps.format_params(3.4e7) == "34.0M"
    sweeps.write_csv(rows, tmp_path / "gpu.csv")
    assert (tmp_path / "gpu.csv").read_text().splitlines()[0].startswith("run_name,size")
    run = next(r for r in runs if r.name == "dana-star-mk4_h8_lr1.0")
    st = sweeps.optimizer_statistics(run)
    np.testing.assert_allclose(st["optimizer/kappa_factor_schedule"]["theory"], st["optimizer/kappa_factor_schedule"]["value"])
    a = st["optimizer/alpha_schedule"]
    assert np.all(a["value"] <= a["theory"] + 1e-12) and a["value"][-1] < a["theory"][-1] or a["value"][-1] == pytest.approx(a["theory"][-1])
    sw = sweeps.kappa_sweep(runs, 8)
    assert list(sw) == [(2.0, 0.85)] and sweeps.adamw_baseline(runs, 8)["final"] == pytest.approx(best[8]["final_loss"])
    assert sweeps.kappa_slices(sw, tenths_only=False) == {2.0: {"kappa": [0.85], "final": [sw[(2.0, 0.85)]["final"]]}}
    assert sweeps.kappa_slices(sw) == {}


def test_hoyer_points_group_by_coefficient():
    runs = [Run(f"r{i}", f"r{i}", {"opt": "adamw", "n_head": 6, "hoyer_loss_coeff": c, "iterations": 100, "batch_size": 4, "acc_steps": 2,
                                   "sequence_length": 512}, {"final-val/loss": l, "iter": 100, "train/hoyer_loss": 0.3})
            for i, (c, l) in enumerate([(0.0, 3.5), (1e-4, 3.45), (1e-4, 3.48), (1e-2, 3.7)])]
    pts = sweeps.hoyer_points(runs)
    assert pts[0]["pf_days"] == pytest.approx(6.0 * sizes.model_size(6, "Qwen3_Hoyer").non_emb * 4096 * 100 / (1e15 * 86400))
    by = sweeps.hoyer_loss_by_coefficient(pts)
    assert [(p["hoyer_coeff"], p["final_val_loss"]) for p in by[(6, "adamw")]] == [(0.0, 3.5), (1e-4, 3.45), (1e-2, 3.7)]


def test_command_line_writes_reports_and_figures(runs_root, tmp_path, capsys):
    from adana_b200.studies.__main__ import main

    assert main(["sizes", "--sizes", "36", "--formula", "6N2"]) == 0
    assert "non_emb 1,719,926,784" in capsys.readouterr().out
    assert main(["lr-law", str(runs_root), "--opt", "adamw", "--omega", "4", "--top-k", "2", "--bootstrap", "10",
                 "--json", str(tmp_path / "law.json"), "--svg", str(tmp_path / "law.svg")]) == 0
    law = json.loads((tmp_path / "law.json").read_text())
    assert law["fit"]["d"] < 0 and law["bootstrap"]["n_valid_samples"] > 0 and (tmp_path / "law.svg").read_text().startswith("<svg")
    assert main(["curvature", str(runs_root), "--opt", "dana-star-mk4", "--json", str(tmp_path / "cur.json"), "--svg", str(tmp_path / "cur.svg")]) == 0
    assert json.loads((tmp_path / "cur.json").read_text())["average_curvature"]["mean"] == pytest.approx(0.05, rel=1e-3)
    assert main(["loss-laws", str(runs_root), "--opts", "adamw", "dana-star-mk4", "--form", "single", "--baseline", "adamw",
                 "--json", str(tmp_path / "laws.json"), "--svg", str(tmp_path / "laws.svg"), "--cache", str(tmp_path / "c")]) == 0
    laws = json.loads((tmp_path / "laws.json").read_text())
    assert np.mean(laws["multiplier"]["dana-star-mk4"][1]) == pytest.approx(1.4, rel=0.1)
    assert main(["gpu-hours", str(runs_root), "--opt", "adamw", "--csv", str(tmp_path / "g.csv")]) == 0
    assert main(["size-curves", str(runs_root), "--opt", "adamw", "--svg", str(tmp_path / "sz.svg")]) == 0
    assert main(["opt-stats", str(runs_root / "dana-star-mk4_h8_lr1.0"), "--svg-prefix", str(tmp_path / "st")]) == 0
    assert (tmp_path / "st_alpha_schedule.svg").exists()
    assert main(["kappa", str(runs_root), "--n-head", "8", "--svg-prefix", str(tmp_path / "k"), "--json", str(tmp_path / "k.json")]) == 0
    assert (tmp_path / "k_curves.svg").exists()
    # compute saved: every size's best candidate run reaches the baseline's final loss by its own end at the latest
    assert main(["savings", str(runs_root), "--opt", "dana-star-mk4", "--baseline", "adamw", "--window", "0", "1e9",
                 "--json", str(tmp_path / "sv.json"), "--svg", str(tmp_path / "sv.svg")]) == 0
    sv = json.loads((tmp_path / "sv.json").read_text())
    assert [r["size"] for r in sv["per_size"]] == [8, 12, 16] and all(r["compute_saved"] >= 0 for r in sv["per_size"])
    assert sv["lines"]["curves"]["dana-star-mk4"]["n_points"] == 3
    # sensitivity from the two reports written above
    assert main(["lr-law", str(runs_root), "--opt", "dana-star-mk4", "--omega", "4", "--top-k", "2", "--bootstrap", "10",
                 "--extrapolate", "16", "--json", str(tmp_path / "law2.json")]) == 0
    assert main(["lr-law", str(runs_root), "--opt", "adamw", "--omega", "4", "--top-k", "2", "--bootstrap", "10",
                 "--extrapolate", "16", "--json", str(tmp_path / "law1.json")]) == 0
    assert main(["sensitivity", "--bootstrap", str(tmp_path / "law1.json"), str(tmp_path / "law2.json"), "--names", "adamw",
                 "dana-star-mk4", "--curvature", str(tmp_path / "cur.json"), "--law", "2.0", "3.0", "0.2", "--losses", "4.9", "4.8",
                 "--target-size", "16", "--json", str(tmp_path / "se.json")]) == 0
    se = json.loads((tmp_path / "se.json").read_text())
    assert [r["optimizer"] for r in se["analysis"]] == ["adamw", "dana-star-mk4"] and "compute_saved" in se["analysis"][1]


def test_gamma3_and_hoyer_commands(tmp_path):
    from adana_b200.studies.__main__ import main

    root = tmp_path / "exps"
    for h in (8, 12):
        for its in (500, 1000, 2000):
            for f in (0.5, 1.0, 2.0):
                g = 2.0 * its ** -0.4 * f
                _write_run(root, f"g_h{h}_{its}_{f}", {"opt": "dana-star-mk4", "n_head": h, "lr": 1e-3, "iterations": its, "gamma_3_factor": g,
                                                       "weight_decay": 0.04, "wd_ts": 100}, 3.0 + abs(math.log(f)), [(its, 3.0)])
    for c, l in ((0.0, 3.5), (1e-4, 3.4), (1e-2, 3.8)):
        _write_run(root, f"hoyer_{c}", {"opt": "adamw", "n_head": 6, "lr": 1e-3, "iterations": 100, "hoyer_loss_coeff": c, "batch_size": 4,
                                        "acc_steps": 1, "sequence_length": 512, "weight_decay": 0.1}, l, [(100, l)])
    assert main(["gamma3", str(root), "--opt", "dana-star-mk4", "--top-k", "1", "--json", str(tmp_path / "g.json"), "--svg", str(tmp_path / "g.svg")]) == 0
    rep = json.loads((tmp_path / "g.json").read_text())
    assert rep["params"] == pytest.approx([2.0, -0.4], rel=1e-6) and len(rep["points"]) == 6
    assert main(["hoyer", str(root), "--opts", "adamw", "--json", str(tmp_path / "h.json"), "--svg", str(tmp_path / "h.svg")]) == 0
    by = json.loads((tmp_path / "h.json").read_text())
    assert [p["hoyer_coeff"] for p in by["6:adamw"]] == [0.0, 1e-4, 1e-2] and (tmp_path / "h.svg").exists()
    curves = (tmp_path / "h_curves.svg").read_text()
    assert curves.count("<polyline") == 3 and "λ=1e-4 (AdamW)" in curves and 'stroke="#000000"' in curves


def test_panels_draw_every_family(tmp_path):
    C = np.geomspace(0.1, 50, 8)
    curves = [{"name": "adamw", "compute": C, "loss": loss_laws.single(C, 1.5, 0.8, 0.2)},
              {"name": "dana-star-mk4", "compute": C, "loss": loss_laws.single(C * 1.3, 1.5, 0.8, 0.2)}]
    fit = loss_laws.fit_joint(curves, "single")
    assert panels.loss_laws(curves, fit, tmp_path / "a.svg").exists()
    fits = {"single": loss_laws.fit_single(C, curves[0]["loss"]), "a=0": loss_laws.fit_single(C, curves[0]["loss"], True)}
    assert "R²" in panels.residuals(fits, C, tmp_path / "b.svg").read_text()
    mult = {"dana-star-mk4": loss_laws.multiplier_piecewise(C, curves[1]["loss"], C, curves[0]["loss"])}
    assert "DANA-Star-MK4" in panels.compute_multiplier(mult, tmp_path / "c.svg").read_text()
    ds = [{"name": "dana-star-mk4", "x": [1.0, 4.0, 9.0, 20.0], "y": [0.3, 1.2, 2.5, 6.0]}]
    assert panels.savings(ds, savings.fit_savings_lines(ds), tmp_path / "d.svg").exists()
    rep = gamma3.study([{"size": s, "iterations": t, "gamma_3_factor": 2.0 * t ** -0.4 * f, "val_loss": 3.0 + abs(math.log(f))}
                        for s in (8, 12) for t in (500, 1000, 2000) for f in (0.5, 1.0, 2.0)], top_k=2)
    assert panels.gamma3(rep, tmp_path / "e.svg").exists()
    by = {(6, "adamw"): [{"hoyer_coeff": c, "final_val_loss": l} for c, l in ((0.0, 3.5), (1e-4, 3.45), (1e-2, 3.7))]}
    assert panels.hoyer(by, tmp_path / "f.svg").exists()


def test_wandb_source_through_the_cache(tmp_path):
    """The W&B source only needs an object with `runs(path, filters)`; the cache keeps what it returned."""
    from types import SimpleNamespace

    from adana_b200.studies.runs import WandbRuns

    calls = []

    class FakeSummary:
        _json_dict = {"final-val/loss": 3.21, "iter": 100}

    class FakeRun(SimpleNamespace):
        def scan_history(self):
            calls.append("history")
            return [{"iter": 50, "val/loss": 3.5}, {"iter": 100, "val/loss": 3.21}]

    class FakeApi:
        def runs(self, path, filters=None):
            calls.append((path, dict(filters or {})))
            return [FakeRun(id="abc123", name="adamw_h8", config={"opt": {"value": "adamw"}, "lr": {"value": 1e-3}, "n_head": 8,
                                                                  "iterations": 100, "weight_decay": 40.0}, summary=FakeSummary())]

    src = CachedRuns(WandbRuns("team", "proj", api=FakeApi()), tmp_path / "c")
    runs = src.fetch({"group": "g1"})
    assert calls == [("team/proj", {"group": "g1"})] and runs[0].opt == "adamw" and runs[0].omega() == pytest.approx(4.0)
    assert runs[0].series("val/loss") == ([50, 100], [3.5, 3.21]) and calls.count("history") == 1
    again = CachedRuns(WandbRuns("team", "proj", api=None), tmp_path / "c").fetch({"group": "g1"})     # no API needed any more
    assert again[0].final_val_loss == 3.21 and again[0].series("val/loss") == ([50, 100], [3.5, 3.21])
    assert (tmp_path / "c" / "history" / "abc123.json").exists()
