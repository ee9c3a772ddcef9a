"""Theory package: NumPy rules vs the PyTorch optimizer classes, convention differences, PLRF risk ODE vs SGD."""
import numpy as np
import pytest
import torch

from adana_b200.optim.logtime import ADana, DanaStarMK4
from adana_b200.theory import (DanaHparams, ODEInputs, PowerLawRF, adana_rule, ademamix_rule, dana_mk4_rule,
                               dana_star_mk4_rule, powerlaw_schedule, scale_by_learning_rate, solve_risk_ode,
                               train_plrf)


def _grads(n, steps, seed=0):
    rng = np.random.default_rng(seed)
    scale = np.geomspace(1e-3, 1.0, n)
    return [rng.standard_normal(n) * scale * (rng.random(n) < 0.6) for _ in range(steps)]


@pytest.mark.parametrize("name", ["adana", "dana-mk4", "dana-star-mk4"])
def test_numpy_rules_reproduce_the_pytorch_classes(name):
    n, steps, lr, kappa, delta = 64, 25, 3e-3, 0.85, 8.0
    rule = {"adana": lambda: adana_rule(kappa=kappa, delta=delta, convention="torch"),
            "dana-mk4": lambda: dana_mk4_rule(kappa=kappa, delta=delta, clipsnr=0.7, convention="torch"),
            "dana-star-mk4": lambda: dana_star_mk4_rule(kappa=kappa, delta=delta, clipsnr=0.7, convention="torch")}[name]()
    init, update = scale_by_learning_rate(rule, lr)
    p = torch.nn.Parameter(torch.linspace(-1, 1, n, dtype=torch.float64))
    cls, kw = {"adana": (ADana, {}), "dana-mk4": (ADana, dict(clipsnr=0.7)),
               "dana-star-mk4": (DanaStarMK4, dict(clipsnr=0.7))}[name]
    opt = cls([p], lr=lr, delta=delta, kappa=kappa, weight_decay=0.0, **kw)
    w = p.detach().numpy().copy()
    state = init(w)
    for g in _grads(n, steps):
        p.grad = torch.from_numpy(g.copy())
        opt.step()
        dw, state = update(g, state, None)
        w = w + dw
        np.testing.assert_allclose(w, p.detach().numpy(), rtol=1e-9, atol=1e-12)


def test_optax_convention_first_step_and_clock():
    g = np.array([0.5, -2.0, 0.0, 1e-3])
    init, update = adana_rule(kappa=0.8, delta=8.0, convention="optax")
    out, st = update(g, init(g), None)
    # count 0: alpha = 1, so m = g, v = g², |m|/sqrt(v) = 1 and the effective time is max(0, 1) = 1
    want = -(g / (np.abs(g) + 1e-8)) - np.sign(g) * (np.abs(g) / (np.abs(g) + 1e-8)) * 2
    np.testing.assert_allclose(out, want, rtol=1e-12)
    assert st.count == 1
    # from the second step on the EMA weight equals the PyTorch one at the same index: (1 + c/delta)^-1 = delta/(delta+c)
    assert np.isclose(1.0 / (1.0 + 3 / 8.0), 8.0 / (8.0 + 3))
    # additive weight decay
    _, update_wd = adana_rule(wd=0.1, convention="optax")
    out_wd, _ = update_wd(g, init(g), np.ones_like(g))
    out_0, _ = adana_rule(convention="optax")[1](g, init(g), np.ones_like(g))
    np.testing.assert_allclose(out_wd - out_0, -0.1 * np.ones_like(g))


def test_star_rule_tau_tracks_activity_rate():
    rng = np.random.default_rng(0)
    init, update = dana_star_mk4_rule(convention="optax")
    w = np.zeros(2)
    st = init(w)
    for _ in range(4000):
        g = np.array([rng.standard_normal(), rng.standard_normal() * (rng.random() < 0.1)])
        _, st = update(g, st, None)
    assert st.tau[0] > 2.5 * st.tau[1] > 0          # the always-on coordinate has the larger tau


def test_ademamix_rule_matches_closed_form_first_steps():
    g = np.array([1.0, -3.0])
    init, update = ademamix_rule(beta1=0.9, beta2=0.99, beta3=0.999, alpha=5.0, gamma_3_factor=0.5, wd=0.0)
    out, st = update(g, init(g), np.zeros(2))
    fast_hat, slow = g, 0.001 * g
    denom = np.sqrt(0.01 * g * g) / np.sqrt(1 - 0.99) + 1e-8
    np.testing.assert_allclose(out, -(fast_hat + 5.0 * 0.5 * slow) / denom, rtol=1e-10)
    init0, update0 = ademamix_rule(beta1=0.0)
    out0, st0 = update0(g, init0(g), None)
    assert st0.fast is None and np.all(np.sign(out0) == -np.sign(g))


def test_powerlaw_schedule():
    s = powerlaw_schedule(1.0, 0.01, -2.0, 100.0)
    assert s(0) == 1.0 and np.isclose(s(100), 0.25) and s(1e6) == 0.01


def test_plrf_problem_identities():
    p = PowerLawRF.initialize_random(1.0, 0.7, 120, 30, seed=3)
    lam, rho = p.hessian_spectrum(), p.rhos()
    # risk at w = 0 splits into the reachable part (sum lambda rho / 2) and the irreducible limit risk
    assert np.isclose(p.population_risk(np.zeros(30)), 0.5 * np.sum(lam * rho) + p.limit_risk(), rtol=1e-10)
    rng = np.random.default_rng(0)
    X, y = p.sample(rng, 200000)
    w = rng.standard_normal(30) * 0.1
    emp = 0.5 * np.mean((X @ w - y) ** 2)
    assert np.isclose(emp, p.population_risk(w), rtol=0.03)


def test_risk_ode_follows_simulated_sgd_and_momentum():
    p = PowerLawRF.initialize_random(1.0, 0.7, 160, 40, seed=1)
    lam, rho = p.hessian_spectrum(), p.rhos()
    z = np.zeros_like(lam)
    inp = ODEInputs(lam, rho, z, z, p.limit_risk())
    lr = 0.5 / p.population_trace
    steps, batch = 1500, 8

    def check(hp, make_rule, tol):
        t, twice = solve_risk_ode(inp, hp, batch=batch, t_max=steps, dt=0.02)
        runs = [train_plrf(p, make_rule(), steps, batch, seed=s) for s in range(6)]
        ts = runs[0][0]
        sim = np.mean([r[1] for r in runs], axis=0)
        for tt, ss in zip(ts, sim):
            if tt >= 50:
                assert abs(np.interp(tt, t, twice) / 2 - ss) / ss < tol, (tt, ss)

    # plain SGD: gradient straight into the parameters
    check(DanaHparams(lambda t: 1.0, lambda t: lr, lambda t: 0.0, lambda t: 1.0),
          lambda: ((lambda w: 0), (lambda g, s, w=None: (-lr * g, s))), 0.12)

    # heavy-ball-like momentum: y <- (1-d) y + g ; w <- w - g2 g - g3 y
    dl, g3 = 0.1, 0.05 * lr

    def momentum_rule():
        def init(w):
            return np.zeros_like(w)

        def update(g, y, w=None):
            y = (1 - dl) * y + g
            return -lr * g - g3 * y, y
        return init, update

    check(DanaHparams(lambda t: 1.0, lambda t: lr, lambda t: g3, lambda t: dl), momentum_rule, 0.15)
    # the approximate ODE (higher-order terms dropped) stays close for small learning rates
    t, full = solve_risk_ode(inp, DanaHparams(lambda t: 1.0, lambda t: 0.2 * lr, lambda t: 0.0, lambda t: 1.0), batch, 500, 0.02)
    _, approx = solve_risk_ode(inp, DanaHparams(lambda t: 1.0, lambda t: 0.2 * lr, lambda t: 0.0, lambda t: 1.0), batch, 500, 0.02,
                               approximate=True)
    assert np.max(np.abs(full - approx) / full) < 0.05


def test_shared_gradient_comparison_and_kappa_sweep():
    from adana_b200.logging.tau_stats import compute_tau_order_statistics
    from adana_b200.theory import compare_rules, final_risk_exponent, sweep, tau_order_statistics

    p = PowerLawRF.initialize_random(1.0, 0.7, 120, 30, seed=2)
    lr = 0.3 / p.population_trace
    rules = {"sgd": ((lambda w: 0), (lambda g, s, w=None: (-lr * g, s))),
             "dana-star-mk4": scale_by_learning_rate(dana_star_mk4_rule(kappa=0.85, clipsnr=2.0), 0.02)}
    res = compare_rules(p, rules, steps=400, batch=8, seed=0)
    assert res["sgd"].shape == res["dana-star-mk4"].shape == res["steps"].shape
    assert res["sgd"][-1] < res["sgd"][0] and res["dana-star-mk4"][-1] < res["dana-star-mk4"][0]
    # same seed -> identical batches: re-running one rule alone reproduces its curve exactly
    alone = compare_rules(p, {"sgd": rules["sgd"]}, steps=400, batch=8, seed=0)
    np.testing.assert_array_equal(alone["sgd"], res["sgd"])
    assert final_risk_exponent(res["steps"], res["sgd"], p.limit_risk()) < 0
    sw = sweep(p, lambda k: scale_by_learning_rate(adana_rule(kappa=k), 0.01), [0.7, 1.0], steps=200, batch=8)
    assert {"0.7", "1", "steps"} <= set(sw)
    tau = res["_final_states"]["dana-star-mk4"].tau
    hi, lo = tau_order_statistics(tau)
    hi2, lo2 = compute_tau_order_statistics(np.asarray(tau))
    np.testing.assert_allclose(hi, hi2)
    np.testing.assert_allclose(lo, lo2)
    assert hi[0] == tau.max() and lo[0] == tau.min()
