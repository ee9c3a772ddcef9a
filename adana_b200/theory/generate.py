"""Data generators of the theory figures: kappa sweeps on the mixture-of-experts PLRF problem ("hummingbird") and
tau order statistics over training time.  Each command trains on CPU with the NumPy rules of `theory/rules.py`,
records every argument next to the results and writes one JSON file; `adana_b200.figures` draws them.

    python -m adana_b200.theory.generate hummingbird --optimizer dana-star-mk4 --steps 20000 --out hummingbird.json
    python -m adana_b200.theory.generate taustats --steps 50000 --out taustats.json
    python -m adana_b200.theory.generate spectra --v 2000 --d 500 --alpha 1.0 --out spectra.json
    python -m adana_b200.theory.generate m-sweep --problem moe --m_range 50,100,200 --steps 20000 --out msweep.json
    python -m adana_b200.theory.generate debug-steps --debug_steps 5 --out trace.json

Same experiments as the reference's jax/hummingbird_generate.py:85-550 (every optimizer sees the same batches, label
noise from a Student-t distribution, learning rates g2 = g2_scale * min(1, batch / Tr K), one run per kappa plus an Adam
baseline) and jax/taustats_generate.py:84-485 (tau of the Dana-Star state at log-spaced times, reduced to order
statistics at ranks floor(1.1^k) from both tails), and the spectral figures of jax/deterministic_equivalent.py.
`m-sweep` trains the first Dana-Star (`rules.dana_star_rule`, kappa = (1 - log_d batch) / (2 alpha) unless given), Dana-Star-MK4 (kappa = 1,
clipped) and Adam on the same batches for several numbers of experts (jax/moe_m_sweeps_mk4.py:414-680) or of classes of
the logistic problem (jax/lr_m_sweeps.py:294-540).  `debug-steps` walks both Dana-Star variants through the first
steps on identical gradients and records the statistics of every buffer (jax/debug_mk4_optimizer.py:15-200).
"""
from __future__ import annotations

import argparse
import json
import time
from typing import Dict

import numpy as np

from .problems import LogisticPLRF, MixtureOfExpertsPLRF, log_spaced_steps, train_logistic_plrf, train_moe_plrf
from .rules import ademamix_rule, dana_mk4_rule, dana_star_mk4_rule, dana_star_rule, scale_by_learning_rate
from .sweeps import tau_order_statistics


class LabelNoiseMoE(MixtureOfExpertsPLRF):
    """Targets get sigma * Student-t(dof) noise (jax/hummingbird_generate.py:27-82)."""

    def __init__(self, *a, student_t_dof: float = 3.0, sigma: float = 0.0, **kw):
        super().__init__(*a, **kw)
        self.dof, self.sigma = student_t_dof, sigma

    def sample_routed(self, rng, batch):
        X, y, e = super().sample_routed(rng, batch)
        if self.sigma:
            y = y + self.sigma * rng.standard_t(self.dof, size=batch)
        return X, y, e


def _problem(a) -> LabelNoiseMoE:
    rng = np.random.default_rng(a.random_seed)
    W = rng.standard_normal((a.v, a.d)) / np.sqrt(a.d)
    return LabelNoiseMoE(a.alpha, a.beta, W, a.m, a.zeta, student_t_dof=a.student_t_dof, sigma=a.sigma)


def adam_rule(lr, beta1=0.9, beta2=0.999, eps=1e-8):
    def init(p):
        z = np.zeros_like(p, dtype=np.float64)
        return (0, z, z.copy())

    def update(g, state, params=None):
        c, m, v = state
        c += 1
        m = beta1 * m + (1 - beta1) * g
        v = beta2 * v + (1 - beta2) * g * g
        return -lr * (m / (1 - beta1 ** c)) / (np.sqrt(v / (1 - beta2 ** c)) + eps), (c, m, v)

    return init, update


def make_rules(a, trace_k: float, steps: int) -> Dict[str, tuple]:
    g2 = a.tanea_lr_scalar * a.g2_scale * min(1.0, a.batch_size / trace_k)
    g3 = a.g3_over_g2 * g2
    kappas = np.arange(a.kappa_min, a.kappa_max + a.kappa_step / 2, a.kappa_step)
    rules = {}
    for k in kappas:
        name = f"{a.optimizer}_kappa{k:.1f}"
        if a.optimizer == "dana-star-mk4":
            rules[name] = dana_star_mk4_rule(g2, g3, a.delta, 1e-8, float(k), a.clipsnr)
        elif a.optimizer == "dana-mk4":
            rules[name] = dana_mk4_rule(g2, g3, a.delta, 1e-8, float(k), a.clipsnr)
        elif a.optimizer == "dana-star":
            rules[name] = dana_star_rule(g2, g3, float(k))
        elif a.optimizer == "ademamix":
            alpha_final, beta3_final = float(steps ** (1.0 - k)), 1.0 - a.delta / steps
            hl = lambda b: np.log(0.5) / np.log(b + 1e-8) - 1.0

            def beta3(c, b1=a.ademamix_beta1, bf=beta3_final):
                p = min(c / steps, 1.0)
                return 0.5 ** (1.0 / ((1 - p) * hl(b1) + p * hl(bf) + 1.0))

            rules[name] = scale_by_learning_rate(
                ademamix_rule(a.ademamix_beta1, a.ademamix_beta2, beta3, lambda c, af=alpha_final: min(c / steps, 1.0) * af),
                a.g2_scale * min(1.0, a.batch_size / trace_k))
        else:
            raise ValueError(f"unknown optimizer {a.optimizer}")
    rules["adam"] = adam_rule(a.adam_lr * min(1.0, a.batch_size / trace_k), a.adam_beta1, a.adam_beta2)
    return rules


def cmd_hummingbird(a):
    prob = _problem(a)
    rules = make_rules(a, prob.population_trace, a.steps)
    out = {"args": vars(a), "traceK": prob.population_trace, "runs": {}}
    t0 = time.time()
    for name, rule in rules.items():
        r = train_moe_plrf(prob, rule, a.steps, a.batch_size, seed=a.random_seed + 1)     # the same batches for every rule
        out["runs"][name] = {"timestamps": r["timestamps"].tolist(), "losses": r["losses"].tolist()}
        print(f"{name}: final risk {r['losses'][-1]:.4e} ({time.time() - t0:.0f}s)")
    return out


def cmd_taustats(a):
    prob = _problem(a)
    g2 = a.tanea_lr_scalar * a.g2_scale * min(1.0, a.batch_size / prob.population_trace)
    init, update = dana_star_mk4_rule(g2, a.g3_over_g2 * g2, a.delta, 1e-8, a.kappa, a.clipsnr)
    times = set(int(t) for t in log_spaced_steps(a.steps, 2.0))
    snapshots = []

    def tracking_update(g, state, params=None):
        d, new = update(g, state, params)
        if new.count in times:
            hi, lo = tau_order_statistics(new.tau)
            snapshots.append({"step": int(new.count), "largest": hi.tolist(), "smallest": lo.tolist(),
                              "mean": float(np.mean(new.tau))})
        return d, new

    r = train_moe_plrf(prob, (init, tracking_update), a.steps, a.batch_size, seed=a.random_seed + 1)
    return {"args": vars(a), "timestamps": r["timestamps"].tolist(), "losses": r["losses"].tolist(),
            "expert_sample_counts": r["expert_sample_counts"].tolist(), "tau": snapshots}


def cmd_spectra(a):
    from . import deterministic as D

    xs, dens = D.spectral_density(a.v, a.d, a.alpha, a.points)
    eigs, rho = D.theory_rhos(a.alpha, a.beta, a.d)
    return {"args": vars(a), "xs": xs.tolist(), "density": dens.tolist(), "kappa": D.theory_kappa(a.alpha, a.v, a.d),
            "lambda_min": D.theory_lambda_min(a.alpha, a.v, a.d), "limit_loss": D.theory_limit_loss(a.alpha, a.beta, a.v, a.d),
            "eigs": eigs.tolist(), "rho": rho.tolist()}


def _star_rules(a, trace_k: float) -> Dict[str, tuple]:
    g2 = a.tanea_lr_scalar * a.g2_scale * min(1.0, a.batch_size / trace_k)
    g3 = a.g3_over_g2 * g2
    kappa_b = np.log(a.batch_size) / np.log(a.d)
    kappa = a.kappa if a.kappa is not None else (1.0 - kappa_b) / (2 * a.alpha)
    rules = {"dana-star": dana_star_rule(g2, g3, float(kappa)),
             "dana-star-mk4": dana_star_mk4_rule(g2, g3, a.delta, 1e-8, 1.0, a.clipsnr)}
    if not a.disable_adam:
        rules["adam"] = adam_rule(a.adam_lr * min(1.0, a.batch_size / trace_k), a.adam_beta1, a.adam_beta2)
    return rules


def cmd_m_sweep(a):
    trace_k = float(np.sum(np.arange(1, a.v + 1, dtype=np.float64) ** (-2.0 * a.alpha)))
    out = {"args": vars(a), "traceK": trace_k, "runs": {}}
    for m in [int(x) for x in str(a.m_range).split(",")]:
        if a.problem == "moe":
            rng = np.random.default_rng(a.random_seed)
            prob = LabelNoiseMoE(a.alpha, a.beta, rng.standard_normal((a.v, a.d)) / np.sqrt(a.d), m, a.zeta,
                                 student_t_dof=a.student_t_dof, sigma=a.sigma)
            train = lambda rule: train_moe_plrf(prob, rule, a.steps, a.batch_size, seed=a.random_seed + 1)
        else:
            prob = LogisticPLRF(a.alpha, a.beta, a.zeta, a.snr, a.v, a.d, m, seed=a.random_seed)
            train = lambda rule: train_logistic_plrf(prob, rule, a.steps, a.batch_size, seed=a.random_seed + 1)
        out["runs"][str(m)] = {}
        for name, rule in _star_rules(a, trace_k).items():
            r = train(rule)
            out["runs"][str(m)][name] = {"timestamps": r["timestamps"].tolist(), "losses": r["losses"].tolist()}
            print(f"m={m} {name}: final risk {r['losses'][-1]:.4e}")
    return out


def buffer_stats(x) -> Dict[str, float]:
    x = np.asarray(x, dtype=np.float64)
    return {"mean": float(x.mean()), "std": float(x.std()), "min": float(x.min()), "max": float(x.max()),
            "norm": float(np.linalg.norm(x))}


def cmd_debug_steps(a):
    """The same gradients through Dana-Star and Dana-Star-MK4: per step the statistics of the gradient, of m, v, tau
    and of the update, so a divergence between the two can be traced to the buffer where it starts."""
    rng = np.random.default_rng(a.random_seed)
    prob = LabelNoiseMoE(a.alpha, a.beta, rng.standard_normal((a.v, a.d)) / np.sqrt(a.d), a.m, a.zeta,
                         student_t_dof=a.student_t_dof, sigma=a.sigma)
    a.disable_adam = True
    rules = _star_rules(a, prob.population_trace)
    data_rng = np.random.default_rng(a.random_seed + 1)
    params = {k: np.zeros((a.d, a.m)) for k in rules}
    states = {k: r[0](params[k]) for k, r in rules.items()}
    trace = []
    for step in range(1, a.debug_steps + 1):
        X, y, experts = prob.sample_routed(data_rng, a.batch_size)
        row = {"step": step}
        for k, (_, update) in rules.items():
            G, _ = prob.routed_gradient(params[k], X, y, experts)
            upd, states[k] = update(G, states[k], params[k])
            params[k] = params[k] + upd
            st = states[k]
            row[k] = {"gradient": buffer_stats(G), "m": buffer_stats(st.m), "v": buffer_stats(st.v), "tau": buffer_stats(st.tau),
                      "update": buffer_stats(upd), "risk": prob.population_risk(params[k])}
            print(f"step {step} {k}: |g| {row[k]['gradient']['norm']:.4e} |m| {row[k]['m']['norm']:.4e} |v| {row[k]['v']['norm']:.4e} "
                  f"tau mean {row[k]['tau']['mean']:.4e} |update| {row[k]['update']['norm']:.4e} risk {row[k]['risk']:.6e}")
        trace.append(row)
    return {"args": vars(a), "trace": trace}


def parser():
    p = argparse.ArgumentParser(prog="python -m adana_b200.theory.generate")
    sub = p.add_subparsers(dest="cmd", required=True)
    for name in ("hummingbird", "taustats", "spectra", "m-sweep", "debug-steps"):
        s = sub.add_parser(name)
        s.add_argument("--alpha", type=float, default=1.0)
        s.add_argument("--beta", type=float, default=0.0 if name != "taustats" else -0.3)
        s.add_argument("--v", type=int, default=2000)
        s.add_argument("--d", type=int, default=500)
        s.add_argument("--out", required=True)
        if name == "spectra":
            s.add_argument("--points", type=int, default=None)
            continue
        if name in ("m-sweep", "debug-steps"):
            s.add_argument("--problem", default="moe", choices=["moe", "logistic"])
            s.add_argument("--m_range", default="50,100,200")
            s.add_argument("--m", type=int, default=100)
            s.add_argument("--zeta", type=float, default=0.5)
            s.add_argument("--snr", type=float, default=1.0)
            s.add_argument("--steps", type=int, default=125000)
            s.add_argument("--debug_steps", type=int, default=5)
            s.add_argument("--batch_size", type=int, default=100)
            s.add_argument("--g2_scale", type=float, default=0.2)
            s.add_argument("--g3_over_g2", type=float, default=0.01)
            s.add_argument("--tanea_lr_scalar", type=float, default=1.0)
            s.add_argument("--kappa", type=float, default=None)
            s.add_argument("--clipsnr", type=float, default=2.0)
            s.add_argument("--delta", type=float, default=8.0)
            s.add_argument("--student_t_dof", type=float, default=3.0)
            s.add_argument("--sigma", type=float, default=0.1)
            s.add_argument("--adam_lr", type=float, default=0.2)
            s.add_argument("--adam_beta1", type=float, default=0.99)
            s.add_argument("--adam_beta2", type=float, default=0.999)
            s.add_argument("--disable_adam", action="store_true")
            s.add_argument("--random_seed", type=int, default=42)
            continue
        s.add_argument("--m", type=int, default=100 if name == "hummingbird" else 1000)
        s.add_argument("--zeta", type=float, default=0.5 if name == "hummingbird" else 1.0)
        s.add_argument("--steps", type=int, default=125000 if name == "hummingbird" else 1000000)
        s.add_argument("--batch_size", type=int, default=100)
        s.add_argument("--g2_scale", type=float, default=0.5)
        s.add_argument("--g3_over_g2", type=float, default=1.0)
        s.add_argument("--tanea_lr_scalar", type=float, default=1.0)
        s.add_argument("--clipsnr", type=float, default=2.0)
        s.add_argument("--delta", type=float, default=8.0)
        s.add_argument("--student_t_dof", type=float, default=3.0)
        s.add_argument("--sigma", type=float, default=0.1 if name == "hummingbird" else 0.0)
        s.add_argument("--random_seed", type=int, default=42)
        if name == "hummingbird":
            s.add_argument("--optimizer", default="dana-star-mk4", choices=["dana-star-mk4", "dana-mk4", "dana-star", "ademamix"])
            s.add_argument("--kappa_min", type=float, default=0.0)
            s.add_argument("--kappa_max", type=float, default=1.0)
            s.add_argument("--kappa_step", type=float, default=0.1)
            s.add_argument("--ademamix_beta1", type=float, default=0.9)
            s.add_argument("--ademamix_beta2", type=float, default=0.999)
            s.add_argument("--adam_lr", type=float, default=0.2)
            s.add_argument("--adam_beta1", type=float, default=0.99)
            s.add_argument("--adam_beta2", type=float, default=0.999)
        else:
            s.add_argument("--kappa", type=float, default=1.0)
    return p


def main(argv=None):
    a = parser().parse_args(argv)
    result = {"hummingbird": cmd_hummingbird, "taustats": cmd_taustats, "spectra": cmd_spectra, "m-sweep": cmd_m_sweep,
              "debug-steps": cmd_debug_steps}[a.cmd](a)
    with open(a.out, "w") as f:
        json.dump(result, f)
    print(f"wrote {a.out}")
    return result


if __name__ == "__main__":
    main()
