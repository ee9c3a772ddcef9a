"""The deterministic equivalent, the mixture-of-experts / logistic problems and the sweep generators of the theory
package (NumPy restatements of the reference's jax/ files; JAX is not installed, so the checks are internal
consistency: fixed points satisfy their equations, densities integrate to what they must, training reduces risk)."""
import json

import numpy as np
import pytest

from adana_b200 import theory as T
from adana_b200.theory import deterministic as D
from adana_b200.theory import generate as G


def test_kappa_tau_and_limit_loss_satisfy_their_fixed_points():
    from scipy.integrate import quad

    alpha, V, Dm = 1.0, 2000, 200
    k = D.theory_kappa(alpha, V, Dm)
    assert abs(k * quad(lambda x: 1.0 / (k + x ** (2 * alpha)), 0.0, V / Dm)[0] - 1.0) < 2e-3
    alpha2 = 0.3
    t = D.theory_tau(alpha2, V, Dm)
    j = np.arange(1, V, dtype=np.float64) ** (2 * alpha2)
    assert abs(t * np.sum(1.0 / (Dm * (j + t))) - 1.0) < 2e-3
    # the limit loss decreases with the sketch dimension and is below the risk at initialisation
    l1, l2 = D.theory_limit_loss(1.0, 0.5, 2000, 100), D.theory_limit_loss(1.0, 0.5, 2000, 400)
    init = 0.5 * np.sum(np.arange(1, 2000.0) ** (-2.0 * 1.5))
    assert 0 < l2 < l1 < init
    assert D.theory_lambda_min(1.0, 2000, 200) > 0


def test_fixed_point_m_solves_its_equation_and_matches_a_random_sketch():
    v, d, alpha = 400, 100, 1.0
    xs = np.geomspace(2e-4, 0.9, 60)
    eps = 1e-3
    m = D.theory_m(v, d, alpha, xs, eta=np.log10(eps), eta_steps=80)
    lam = np.arange(1, v + 1.0) ** (-2 * alpha)
    z = xs + 1j * eps
    resid = m + (lam[:, None] * m / (lam[:, None] * m - z)).sum(0) / d - 1.0
    assert np.abs(resid).max() < 1e-3          # (one Newton step per rung of the ladder, as in the reference)
    # the limit loss of the deterministic equivalent predicts the least-squares risk of an actual random sketch
    prob = T.PowerLawRF.initialize_random(alpha, 0.4, v, d, seed=1)
    assert abs(prob.limit_risk() / D.theory_limit_loss(alpha, 0.4, v, d) - 1.0) < 0.35
    # the density of states integrates to ~d eigenvalues (mass d / 1 per eigenvalue)
    grid, dens = D.spectral_density(v, d, alpha, 4000)
    mass = np.trapezoid(dens, grid)
    assert 0.6 * d < mass < 1.4 * d, mass


def test_moe_and_logistic_problems_train():
    prob = T.MixtureOfExpertsPLRF.initialize_random(1.0, 0.3, 120, 30, m=6, zeta=1.0, seed=0)
    assert abs(prob.expert_probs.sum() - 1) < 1e-12 and prob.expert_probs[0] > prob.expert_probs[-1]
    g2 = 0.5 * min(1.0, 20 / prob.population_trace)
    r = T.train_moe_plrf(prob, T.dana_star_mk4_rule(g2, g2, kappa=0.8), steps=300, batch=20, track_per_expert=True,
                         track_counts=True)
    assert r["losses"][-1] < 0.5 * r["losses"][0]
    assert r["expert_sample_counts"].sum() == 300 * 20
    assert r["expert_sample_counts"][0] > r["expert_sample_counts"][-1]            # power-law routing
    assert (r["expert_update_counts"] <= 300).all() and r["per_expert_losses"].shape[1] == 6
    # the frequent expert is further along than the rare one
    assert r["per_expert_losses"][-1][0] < r["per_expert_losses"][-1][-1]
    two = T.MixtureOfExpertsPLRF.two_experts(1.0, 0.3, 80, 20, p=0.1)
    assert np.allclose(two.expert_probs, [0.9, 0.1])
    lp = T.LogisticPLRF(1.0, 0.5, 1.0, snr=4.0, v=100, d=24, m=8, seed=0, eval_samples=2000)
    out = T.train_logistic_plrf(lp, G.adam_rule(0.05), steps=200, batch=32)
    assert out["losses"][0] == np.float64(np.log(8)).item() or abs(out["losses"][0] - np.log(8)) < 1e-9
    assert out["losses"][-1] < out["losses"][0] - 0.2


def test_generators_write_their_json(tmp_path):
    h = G.main(["hummingbird", "--v", "120", "--d", "30", "--m", "6", "--steps", "150", "--kappa_step", "0.5",
                "--out", str(tmp_path / "h.json")])
    assert set(h["runs"]) == {"dana-star-mk4_kappa0.0", "dana-star-mk4_kappa0.5", "dana-star-mk4_kappa1.0", "adam"}
    t = G.main(["taustats", "--v", "120", "--d", "30", "--m", "12", "--steps", "130", "--out", str(tmp_path / "t.json")])
    assert [s["step"] for s in t["tau"]][:4] == [2, 4, 8, 16] and len(t["tau"][-1]["largest"]) > 5
    assert max(t["tau"][-1]["largest"]) <= 1.0 and min(t["tau"][-1]["smallest"]) >= 0.0
    s = G.main(["spectra", "--v", "300", "--d", "60", "--out", str(tmp_path / "s.json")])
    assert s["kappa"] > 0 and s["lambda_min"] > 0 and len(s["xs"]) == len(s["density"])
    assert json.loads((tmp_path / "s.json").read_text())["limit_loss"] == s["limit_loss"]


# ---- schedule experiments on the risk ODE ------------------------------------------------------------------------------
def test_ode_options_momentum_renormalisation_and_dynamic_g3():
    from adana_b200.theory import schedule_studies as S
    from adana_b200.theory.ode import DanaHparams, solve_risk_ode

    inp = S.ode_inputs(0.7, 0.5, 320, 80)
    lr = min(1.0, 1 / S.population_trace(0.7, 320))
    hp = DanaHparams(S.const(1.0), S.const(0.5 * lr), S.const(0.05 * lr), S.delta_schedule(0.7, 0.5))
    t0, r0 = solve_risk_ode(inp, hp, 1, 1e3, 2e-2)
    t1, r1, m1 = solve_risk_ode(inp, hp, 1, 1e3, 2e-2, momentum=True)
    np.testing.assert_array_equal(r0, r1)                     # asking for the momentum does not change the risk
    assert m1[0] == 0.0 and np.all(m1[1:] > 0) and len(m1) == len(t1)
    _, r_ratio, m_ratio = solve_risk_ode(inp, hp, 1, 1e3, 2e-2, momentum=True, dynamic_g3="ratio")
    sgd = DanaHparams(hp.g1, hp.g2, S.const(0.0), hp.delta)
    _, r_sgd = solve_risk_ode(inp, sgd, 1, 1e3, 2e-2)
    # this constant g3 is too large for a raw-sum momentum: ungated the risk turns around and grows; gated by
    # min(R / ||y||^2, 1) it keeps falling and ends next to SGD
    assert r0[-1] > 10 * r_sgd[-1] and r_ratio[-1] == pytest.approx(r_sgd[-1], rel=0.05) and np.all(np.diff(r_ratio) < 0)
    _, r_star = solve_risk_ode(inp, hp, 1, 1e3, 2e-2, risk_renormalized=True)
    assert r_star[-1] != r0[-1] and np.all(np.isfinite(r_star))
    shifted = solve_risk_ode(inp, DanaHparams(hp.g1, hp.g2, hp.g3, lambda t: 1.0 / (1.0 + t)), 1, 1e2, 2e-2, shifted_clock=True)[1]
    plain = solve_risk_ode(inp, DanaHparams(hp.g1, hp.g2, hp.g3, lambda t: 1.0 / (2.0 + t)), 1, 1e2, 2e-2)[1]
    np.testing.assert_allclose(shifted, plain, rtol=1e-12)   # delta read one step later == the schedule shifted by one


def test_optimizer_comparison_on_the_ode():
    from adana_b200.theory import schedule_studies as S

    r = S.compare_optimizers(alpha=1.2, d=80, steps=2e4, dt=2e-2)
    final = {k: v["loss"][-1] for k, v in r["runs"].items()}
    assert set(final) == {"sgd", "dana-constant", "dana-decay", "ademamix"}
    assert all(r["risk_infinity"] < f < v["loss"][0] for f, v in zip(final.values(), r["runs"].values()))
    assert final["dana-decay"] < final["sgd"] and final["dana-constant"] < final["sgd"]
    assert r["runs"]["sgd"]["t"][0] == 1.0


def test_kappa_sweep_checkpoints_and_self_consistent_kappa():
    from adana_b200.theory import schedule_studies as S

    ks = np.linspace(0, 1, 6, endpoint=False)
    r = S.kappa_sweep(alpha=0.5, d=80, v=320, steps=1e4, dt=2e-2, kappas=ks)
    assert sorted(r["checkpoints"]) == [10, 100, 1000, 10000] and len(r["runs"]) == 6
    last = r["checkpoints"][10000]
    assert last["best_kappa"] in ks and 0.0 <= last["effective_kappa"] <= 1.0
    np.testing.assert_allclose(last["risk_exponent"], np.log(last["risk"]) / np.log(1e4))
    # later in training a smaller growth exponent is the better one: the schedule must not keep growing like t
    assert r["checkpoints"][10000]["best_kappa"] < r["checkpoints"][100]["best_kappa"]
    res = S.alpha_crossings([0.7, 0.95, 1.2], d=100, v=400, steps=1e5, dt=2e-2, kappas=np.linspace(-1.5, -0.2, 14, endpoint=False))
    k = [row["kappa"] for row in res["rows"]]
    assert all(x is not None and -1.5 < x < -0.2 for x in k) and k[0] < k[1] < k[2]      # flatter spectra want faster decay
    assert res["fit"]["r_squared"] > 0.99 and res["fit"]["slope"] < 0


def test_dynamic_and_danastar_schedule_runs():
    from adana_b200.theory import schedule_studies as S

    plain = S.dynamic_schedules(alpha=0.7, d=100, v=400, steps=1e4, dt=2e-2)
    star = S.danastar_schedules(alpha=0.7, d=100, v=400, steps=1e4, dt=2e-2)
    for r in (plain, star):
        assert set(r["runs"]) == {"dana-constant", "dana-decay", "sgd", "dynamic"}
        for run in r["runs"].values():
            assert np.all(np.isfinite(run["risk"])) and run["risk"][-1] < run["risk"][0]
    assert np.all(plain["runs"]["sgd"]["momentum"][1:] > 0)        # momentum is tracked even when it is not used
    assert star["runs"]["sgd"]["late_slope"] < 0


def test_schedule_studies_and_generators_command_lines(tmp_path):
    from adana_b200.theory import generate, schedule_studies as S

    assert S.main(["compare", "--alpha", "1.2", "--d", "40", "--steps", "2000", "--dt", "0.05", "--out", str(tmp_path / "c.json"),
                   "--svg", str(tmp_path / "c.svg")]) == 0
    assert set(json.loads((tmp_path / "c.json").read_text())["runs"]) == {"sgd", "dana-constant", "dana-decay", "ademamix"}
    assert (tmp_path / "c.svg").read_text().count("<polyline") == 4
    assert S.main(["crossing", "--alphas", "0.8", "1.1", "--d", "60", "--steps", "20000", "--dt", "0.05", "--num-kappa", "10",
                   "--out", str(tmp_path / "x.json"), "--svg", str(tmp_path / "x.svg")]) == 0
    assert S.main(["dynamic", "--danastar", "--d", "40", "--steps", "2000", "--dt", "0.05", "--out", str(tmp_path / "d.json")]) == 0
    res = generate.main(["m-sweep", "--problem", "moe", "--m_range", "3,6", "--steps", "150", "--v", "120", "--d", "30",
                         "--batch_size", "16", "--out", str(tmp_path / "m.json")])
    assert set(res["runs"]) == {"3", "6"} and set(res["runs"]["3"]) == {"dana-star", "dana-star-mk4", "adam"}
    assert all(run["losses"][-1] < run["losses"][0] for m in res["runs"].values() for run in m.values())
    res = generate.main(["m-sweep", "--problem", "logistic", "--m_range", "4", "--steps", "100", "--v", "60", "--d", "20",
                         "--batch_size", "16", "--disable_adam", "--out", str(tmp_path / "l.json")])
    assert set(res["runs"]["4"]) == {"dana-star", "dana-star-mk4"}
    dbg = generate.main(["debug-steps", "--debug_steps", "3", "--v", "100", "--d", "30", "--m", "6", "--batch_size", "20",
                         "--out", str(tmp_path / "t.json")])
    first = dbg["trace"][0]
    assert first["dana-star"]["m"] == first["dana-star-mk4"]["m"]            # identical gradients, identical first step
    assert set(first["dana-star"]) == {"gradient", "m", "v", "tau", "update", "risk"}
    assert dbg["trace"][-1]["dana-star"]["risk"] < 0.5 * 1.0 + 1.0


def test_first_dana_star_rule_against_a_scalar_restatement():
    """`dana_star_rule` (the first Dana-Star of the JAX package) against the same formulas written out per coordinate
    with plain floats, including the effective time max(tau t, 1) at which each coordinate reads its own g3."""
    import math

    rng = np.random.default_rng(3)
    g2c, g3c, kappa, eps, clip = 0.05, 0.02, 0.6, 1e-8, 2.0
    init, update = T.dana_star_rule(g2c, g3c, kappa, eps, clip, wd=1e-3)
    p = rng.standard_normal(7)
    state = init(p)
    m, v, tau = [0.0] * 7, [0.0] * 7, [0.0] * 7
    for count in range(12):
        g = rng.standard_normal(7) * (rng.random(7) < 0.6)          # sparse gradients exercise the tau floor
        d, state = update(g, state, p)
        beta = 1.0 / (1.0 + count / 6.0)
        for i in range(7):
            u = float(g[i])
            v[i] = v[i] * (1 - beta) + beta * u * u
            tau[i] = tau[i] * (1 - beta) + beta * abs(u) / (abs(u) + math.sqrt(v[i]) + eps)
            m[i] = m[i] * (1 - beta) + beta * u
            h = min(tau[i], 0.5)
            r = math.sqrt(max(h / (1 - h), 1.0 / (1.0 + count)))
            eff = max(tau[i] * count, 1.0)
            g3 = g3c * (1.0 + eff) ** (1.0 - kappa)
            scale = r / (math.sqrt(v[i]) + eps)
            want = -g2c * u * scale * min(1.0, clip * math.sqrt(v[i]) / (r * abs(u) + eps)) - g3 * m[i] * scale - 1e-3 * p[i]
            assert d[i] == pytest.approx(want, rel=1e-12, abs=1e-15), (count, i)
        p = p + d
    assert state.count == 12
