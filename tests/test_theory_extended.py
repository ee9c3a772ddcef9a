"""The deterministic equivalent, the mixture-of-experts / logistic problems and the sweep generators of the theory
package (NumPy restatements of the reference's jax/ files; JAX is not installed, so the checks are internal
consistency: fixed points satisfy their equations, densities integrate to what they must, training reduces risk)."""
import json

import numpy as np

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
    grid, dens = D.deterministic_spectra(v, d, alpha, 4000)
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
