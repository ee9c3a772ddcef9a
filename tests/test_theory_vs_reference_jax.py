"""The NumPy theory package against the reference's own JAX files.  `benchmarks/reference_jax_oracle.py` imports
`jax/optimizers.py` and `jax/deterministic_equivalent.py` of the reference unmodified on top of stand-in `jax` / `optax`
modules that map the few calls they make onto NumPy, and records parameter trajectories and theory values in
`tests/golden/theory_reference_values.json`; here the restatements in `adana_b200/theory` must reproduce them."""
import json
from pathlib import Path

import numpy as np
import pytest

from adana_b200 import theory as T
from adana_b200.theory import deterministic as D

G = json.loads((Path(__file__).parent / "golden" / "theory_reference_values.json").read_text())
LR = lambda c: 0.5 / (1.0 + c / 20.0)


def _trajectory(rule, grads, p0):
    init, update = T.scale_by_learning_rate(rule, LR)
    p = np.array(p0, dtype=np.float64)
    state = init(p)
    out = []
    for g in grads:
        d, state = update(np.asarray(g), state, p)
        p = p + d
        out.append(p.copy())
    return np.array(out)


def _rule(name, kw):
    if name.startswith("adana"):
        return T.adana_rule(kw["g2_constant"], kw["g3_constant"], kw["delta"], 1e-8, kw["kappa"])
    if name.startswith("dana_mk4"):
        return T.dana_mk4_rule(kw["g2_constant"], kw["g3_constant"], kw["delta"], 1e-8, kw["kappa"], kw["clipsnr"])
    if name.startswith("dana_star_mk4"):
        return T.dana_star_mk4_rule(kw["g2_constant"], kw["g3_constant"], kw["delta"], 1e-8, kw["kappa"], kw["clipsnr"])
    if name.startswith("dana_star"):
        return T.dana_star_rule(kw["g2_constant"], kw["g3_constant"], kw["kappa_exponent"])
    if name == "ademamix":
        return T.ademamix_rule(0.9, 0.99, lambda c: 1.0 - 0.1 / (1.0 + c / 10.0), lambda c: min(c / 20.0, 1.0) * 3.0, 0.7, 1e-8, 0.01)
    raise KeyError(name)


@pytest.mark.parametrize("name", sorted(G["rules"]["runs"]))
def test_update_rules_follow_the_reference_jax_trajectories(name):
    """Forty steps on a partly sparse gradient sequence (the tau estimator sees zeros, the SNR clip engages in the
    tight-clip cases): every parameter after every step equals the reference optimizer's, to rounding."""
    run = G["rules"]["runs"][name]
    mine = _trajectory(_rule(name, run["kwargs"]), G["rules"]["grads"], G["rules"]["p0"])
    want = np.array(run["params"])
    assert mine.shape == want.shape == (40, 6)
    np.testing.assert_allclose(mine, want, rtol=1e-9, atol=1e-12)
    assert np.abs(want[-1] - np.array(G["rules"]["p0"])).max() > 1e-3          # the trajectories actually move


def test_powerlaw_schedule_matches():
    g = G["powerlaw_schedule"]
    s = T.powerlaw_schedule(*g["args"])
    np.testing.assert_allclose([float(s(t)) for t in g["t"]], g["values"], rtol=1e-12)


def test_deterministic_equivalent_scalars_match():
    d = G["deterministic"]
    for c in d["limit_loss"]:
        assert D.theory_limit_loss(*c["args"]) == pytest.approx(c["value"], rel=2e-3)     # kappa / tau inside are iterated to 1e-3
    for c in d["kappa"]:
        assert D.theory_kappa(*c["args"]) == pytest.approx(c["value"], rel=2e-3)
    for c in d["tau"]:
        assert D.theory_tau(*c["args"]) == pytest.approx(c["value"], rel=2e-3)
    for c in d["lambda_min"]:
        assert D.theory_lambda_min(*c["args"]) == pytest.approx(c["value"], rel=1e-4)
    for c in d["rhos"]:
        eigs, rho = D.theory_rhos(*c["args"])
        np.testing.assert_allclose(eigs, c["eigs"], rtol=1e-10)
        np.testing.assert_allclose(rho, c["rho"], rtol=1e-10)
    cw = d["chunk_weights"]
    np.testing.assert_allclose(D.chunk_weights(np.array(cw["xs"]), np.array(cw["density"]), np.array(cw["a"]), np.array(cw["b"])),
                               cw["value"], rtol=1e-10)


def test_fixed_point_and_measures_match():
    d = G["deterministic"]
    m = d["m"]
    want = np.array(m["value"]["re"]) + 1j * np.array(m["value"]["im"])
    got = D.theory_m(m["args"]["v"], m["args"]["d"], m["args"]["alpha"], np.array(m["xs"]))
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-9)
    f = d["f_measure"]
    np.testing.assert_allclose(D.theory_f_measure(f["args"]["v"], f["args"]["d"], f["args"]["alpha"], f["args"]["beta"], np.array(f["xs"])),
                               f["value"], rtol=1e-5, atol=1e-9)
    e = d["empirical_measure"]
    np.testing.assert_allclose(D.theory_empirical_measure(e["args"]["v"], e["args"]["d"], e["args"]["alpha"], np.array(e["xs"])),
                               e["value"], rtol=1e-5, atol=1e-9)


def _ode_setup():
    from adana_b200.theory.ode import DanaHparams, ODEInputs

    o = G["ode"]
    a = o["args"]
    eigs, rho = D.theory_rhos(a["alpha"], a["beta"], a["d"])
    z = np.zeros_like(rho)
    inp = ODEInputs(eigs, rho, z, z.copy(), o["risk_infinity"])
    dl = T.powerlaw_schedule(1.0, 0.0, -1.0, 6.0)
    return o, a, inp, dl, DanaHparams


@pytest.mark.parametrize("name,kw", [("full", {}), ("approximate", dict(approximate=True)), ("adam", dict(adaptive="adam")),
                                     ("rmsprop_dana", dict(adaptive="rmsprop_dana"))])
def test_risk_ode_equals_the_reference_solver(name, kw):
    """`solve_risk_ode` against `ode_resolvent_log_implicit` of the reference's jax/dana_plrf.py, run unmodified on the
    NumPy stand-in: the full and the approximate coefficients and both adaptive normalisations."""
    o, a, inp, dl, DanaHparams = _ode_setup()
    hp = DanaHparams(lambda t: 1.0, lambda t: 0.05, T.powerlaw_schedule(0.02, 0.0, -0.5, 1.0), dl)
    t, r = T.solve_risk_ode(inp, hp, a["batch"], a["t_max"], a["dt"], **kw)
    want = o["runs"][name]
    np.testing.assert_allclose(t, want["t"], rtol=1e-5, atol=1e-6)        # the reference keeps its time grid in float32
    np.testing.assert_allclose(r, want["twice_risk"], rtol=2e-4)
    assert r[-1] < 0.05 * r[0]


def test_momentum_tracking_and_trajectory_driven_schedules_equal_the_reference_variants():
    """The options of `solve_risk_ode` against the solver copies inside jax/kappa_sweep_plot.py (momentum norm, DanaStar
    renormalisation, the power rule for g3) and jax/dynamical_schedule_plot.py (the ratio rule)."""
    o, a, inp, dl, DanaHparams = _ode_setup()
    hp = DanaHparams(dl, lambda t: 0.01, T.powerlaw_schedule(0.01, 0.0, 0.4, 1.0), dl)
    for name, kw in (("momentum_renormalized", dict(risk_renormalized=True)), ("momentum_plain", {}),
                     ("momentum_dynamic", dict(risk_renormalized=True, dynamic_g3=(0.0, 0.75, 1.0)))):
        t, r, m = T.solve_risk_ode(inp, hp, a["batch"], a["t_max"], a["dt"], momentum=True, shifted_clock=True, **kw)
        want = o["runs"][name]
        np.testing.assert_allclose(r, want["twice_risk"], rtol=2e-4, err_msg=name)
        np.testing.assert_allclose(m, want["momentum"], rtol=2e-3, atol=1e-12, err_msg=name)
    hp = DanaHparams(lambda t: 1.0, lambda t: 0.05, lambda t: 0.02, dl)
    t, r, m = T.solve_risk_ode(inp, hp, a["batch"], a["t_max"], a["dt"], momentum=True, dynamic_g3="ratio")
    want = o["runs"]["ratio_rule"]
    np.testing.assert_allclose(r, want["twice_risk"], rtol=2e-4)
    np.testing.assert_allclose(m, want["momentum"], rtol=2e-3, atol=1e-12)


def test_deterministic_spectrum_and_rho_weights_match():
    """Eigenvalues read off half-integer crossings of the accumulated spectral measure, and the rho weights as contour
    pieces around the leading eigenvalues.  The reference evaluates these in single-precision complex numbers, so the
    densities agree to a few digits and a crossing can land on the neighbouring grid point."""
    s = G["deterministic"]["spectra"]
    got, want = D.deterministic_spectra(**s["args"]), np.array(s["value"])
    assert len(got) == len(want) == s["args"]["d"]
    np.testing.assert_allclose(got, want, rtol=0.03)
    r = G["deterministic"]["rho_weights"]
    got = D.deterministic_rho_weights(**r["args"], a=np.array(r["a"]), b=np.array(r["b"]))
    np.testing.assert_allclose(got, r["value"], rtol=0.03)
    assert np.all(got > 0)


def test_power_law_rf_problem_matches_the_reference_class():
    """The reference's PowerLawRF built on a given sketch W: risk of arbitrary weights, Hessian spectrum, the rho_j of
    the target, the trace that sets the stable step, and the risk of the least-squares solution."""
    g = G["plrf"]
    prob = T.PowerLawRF(g["alpha"], g["beta"], np.array(g["W"]))
    assert prob.population_trace == pytest.approx(g["population_trace"], rel=1e-12)
    for w, want in zip(g["w"], g["risk"]):
        assert prob.population_risk(np.array(w)) == pytest.approx(want, rel=1e-10)
    np.testing.assert_allclose(prob.hessian_spectrum(), g["hessian_spectra"], rtol=1e-9)
    np.testing.assert_allclose(prob.rhos(), g["rhos"], rtol=1e-7)
    assert prob.limit_risk() == pytest.approx(g["empirical_limit_loss"], rel=1e-6)
    assert D.theory_limit_loss(g["alpha"], g["beta"], 60, 12) == pytest.approx(g["theory_limit_loss"], rel=2e-3)


def test_moe_problem_matches_the_reference_class():
    g = G["moe_plrf"]
    prob = T.MixtureOfExpertsPLRF(g["alpha"], g["beta"], np.array(g["W"]), g["m"], g["zeta"])
    np.testing.assert_allclose(prob.expert_probs, g["expert_probs"], rtol=1e-12)
    params = np.array(g["params"])
    assert prob.population_risk(params) == pytest.approx(g["risk"], rel=1e-10)
    np.testing.assert_allclose(prob.per_expert_population_risk(params), g["per_expert"], rtol=1e-10)
    assert T.PowerLawRF.population_risk(prob, params[:, 0]) == pytest.approx(g["single_risk"], rel=1e-10)
    assert prob.limit_risk() == pytest.approx(g["optimal_risk"], rel=1e-6)
    two = T.MixtureOfExpertsPLRF.two_experts(1.0, 0.3, 40, 8, 0.7)
    np.testing.assert_allclose(two.expert_probs, g["two_expert_probs"], rtol=1e-12)


def test_logistic_problem_matches_the_reference_class():
    """The reference's LogisticRegressionPLRF: class frequencies, the scaling of class means and noise, and the
    cross-entropy of given parameters on a batch the reference generated (labels as class indices here)."""
    g = G["logistic_plrf"]
    prob = T.LogisticPLRF(g["alpha"], g["beta"], g["zeta"], g["snr"], g["v"], g["d"], g["m"], seed=0, eval_samples=16)
    np.testing.assert_allclose(prob.class_probs, g["class_probs"], rtol=1e-12)
    np.testing.assert_allclose(prob.noise_std ** 2, g["sigma_eps_diag"], rtol=1e-12)
    assert prob.W.shape == np.array(g["W"]).shape and prob.mu.shape == np.array(g["mu"]).shape
    # the class means carry variance snr * j^(-2 beta) per coordinate in both
    j = np.arange(1, g["v"] + 1.0)
    assert np.mean(np.array(g["mu"]) ** 2 / (g["snr"] * j ** (-2 * g["beta"]))[:, None]) == pytest.approx(1.0, rel=0.5)
    assert np.mean(prob.mu ** 2 / (g["snr"] * j ** (-2 * g["beta"]))[:, None]) == pytest.approx(1.0, rel=0.5)
    params = (np.array(g["theta"]), np.array(g["bias"]))
    X, c = np.array(g["X"]), np.array(g["classes"])
    assert prob.cross_entropy(params, X, c) == pytest.approx(g["cross_entropy"], rel=1e-6)
    # and the analytic gradient used in training is the gradient of that loss
    g_theta, g_b = prob.gradient(params, X, c)
    eps = 1e-6
    bumped = (params[0].copy(), params[1].copy())
    bumped[0][2, 3] += eps
    assert (prob.cross_entropy(bumped, X, c) - prob.cross_entropy(params, X, c)) / eps == pytest.approx(g_theta[2, 3], rel=1e-4)
    bumped = (params[0].copy(), params[1].copy())
    bumped[1][1] += eps
    assert (prob.cross_entropy(bumped, X, c) - prob.cross_entropy(params, X, c)) / eps == pytest.approx(g_b[1], rel=1e-4)


@pytest.mark.parametrize("optimizer", ["dana-star-mk4", "dana-mk4", "dana-star", "ademamix"])
def test_sweep_generator_builds_the_same_optimizers_as_the_reference_generator(optimizer):
    """`theory.generate.make_rules` against `create_optimizers` of the reference's jax/hummingbird_generate.py: the
    constants derived from batch size and trace, one rule per kappa of the grid under the same name, AdEMAMix's alpha
    and beta3 warm-ups, and the Adam baseline; every rule is driven over the same gradients."""
    from types import SimpleNamespace

    from adana_b200.theory import generate

    g = G["hummingbird_rules"]
    rules = generate.make_rules(SimpleNamespace(optimizer=optimizer, **g["args"]), g["traceK"], g["steps"])
    want = g["runs"][optimizer]
    assert sorted(rules) == sorted(want)
    for name, rule in rules.items():
        init, update = rule
        p = np.array(g["p0"])
        state = init(p)
        out = []
        for grad in g["grads"]:
            d, state = update(np.asarray(grad), state, p)
            p = p + d
            out.append(p.copy())
        # (the reference forms its learning-rate constants in single precision: agreement to 1e-6, not to rounding)
        np.testing.assert_allclose(np.array(out), want[name], rtol=2e-6, atol=1e-7, err_msg=name)


def test_m_sweep_builds_the_same_optimizers_as_the_reference_sweep_script():
    """`theory.generate._star_rules` against `get_dana_star_optimizer`, `get_dana_star_mk4_optimizer` and `get_adam_lr` of
    the reference's jax/moe_m_sweeps_mk4.py: the first Dana-Star at kappa = (1 - log_d batch) / (2 alpha) (or a given
    kappa), Dana-Star-MK4 at kappa 1 with the default clip, Adam's step size."""
    from types import SimpleNamespace

    from adana_b200.theory import generate

    g = G["m_sweep_rules"]

    def run(rule):
        init, update = rule
        p = np.array(g["p0"])
        state, out = init(p), []
        for grad in g["grads"]:
            d, state = update(np.asarray(grad), state, p)
            p = p + d
            out.append(p.copy())
        return np.array(out)

    a = SimpleNamespace(kappa=None, clipsnr=2.0, delta=8.0, disable_adam=False, adam_beta1=0.99, adam_beta2=0.999, **g["args"])
    rules = generate._star_rules(a, g["traceK"])
    for name in ("dana-star", "dana-star-mk4"):
        np.testing.assert_allclose(run(rules[name]), g["runs"][name], rtol=2e-6, atol=1e-7, err_msg=name)
    a.kappa = 0.7
    np.testing.assert_allclose(run(generate._star_rules(a, g["traceK"])["dana-star"]), g["runs"]["dana-star_kappa0.7"], rtol=2e-6, atol=1e-7)
    assert g["args"]["adam_lr"] * min(1.0, g["args"]["batch_size"] / g["traceK"]) == pytest.approx(g["adam_lr"], rel=1e-6)


def test_optimizer_comparison_equals_the_reference_script():
    """`schedule_studies.compare_optimizers` against `run_ode` of the reference's jax/plrf_ademamix_behavior.py: SGD,
    Dana with constant and with decaying g3, and AdEMAMix expressed as Dana schedules (g1 = 1/(1+t), alpha and beta3
    warm-ups), all on the deterministic spectrum."""
    from adana_b200.theory import schedule_studies as S

    g = G["optimizer_comparison"]
    c = g["cfg"]
    mine = S.compare_optimizers(c["alpha"], c["beta"], c["d"], c["v"], c["batch_size"], float(c["steps"]), c["lr_scale"], c["g2"],
                                c["g3"], c["delta"], dt=1e-3)
    assert mine["risk_infinity"] == pytest.approx(g["risk_infinity"], rel=2e-3)
    for name, want in g["runs"].items():
        t, loss = mine["runs"][name]["t"][::50], mine["runs"][name]["loss"][::50]
        np.testing.assert_allclose(t, want["t"], rtol=1e-5)
        np.testing.assert_allclose(loss, want["loss"], rtol=3e-3, err_msg=name)       # the floor differs by its own tolerance


def test_exact_lr_law_fit_is_at_least_as_good_as_the_reference_adagrad_fit():
    """The reference fits lr = a (b + P)^d with 6000 Adagrad steps from a fixed start (run here with its own code, the
    gradients taken by differences); `studies.lr_law.fit_weighted` solves the same weighted objective exactly.  The exact
    fit must not be worse on that objective, and inside the range of the data both must predict the same learning rates."""
    from adana_b200.studies import lr_law

    g = G["lr_law_fit"]
    P, lr, w = np.array(g["P"]), np.array(g["lr"]), np.array(g["w"])

    def objective(a, b, d):
        cw = w * w * P
        return float(np.sum(cw * (np.log(lr) - np.log(a * (b + P) ** d)) ** 2) / np.sum(cw))

    a, b, d, err = lr_law.fit_weighted(P, lr, w)
    assert err == pytest.approx(objective(a, b, d), rel=1e-9)
    assert err <= objective(g["a"], g["b"], g["d"]) * (1 + 1e-9)
    grid = np.geomspace(P.min(), P.max(), 20)
    np.testing.assert_allclose(lr_law.predict(grid, a, b, d), g["a"] * (g["b"] + grid) ** g["d"], rtol=0.08)


def test_joint_loss_law_fit_is_at_least_as_good_as_the_reference_adagrad_fit():
    """Two optimizers, one shared floor: the reference's `fit_all_saturated_power_laws_joint` (20 000 Adagrad steps, its
    own code on the stand-ins, gradients by differences) against `studies.loss_laws.fit_joint` on the same objective,
    the mean squared difference of log loss over all points."""
    from adana_b200.studies import loss_laws

    g = G["joint_fit"]

    def objective(fit):
        r = []
        for c in g["curves"]:
            q = fit["curves"][c["name"]]
            pred = loss_laws.broken(np.array(c["compute"]), fit["a"], q["b"], q["c"], q["e"], q["f"])
            r.append(np.log(pred) - np.log(np.array(c["loss"])))
        return float(np.mean(np.concatenate(r) ** 2))

    mine = loss_laws.fit_joint(g["curves"], "broken")
    assert objective(mine) <= objective(g["reference"]) * (1 + 1e-9)
    assert min(q["r_squared"] for q in mine["curves"].values()) >= min(q["r_squared"] for q in g["reference"]["curves"].values()) - 1e-6
    assert 0 < mine["a"] < 0.99 * min(min(c["loss"]) for c in g["curves"])
