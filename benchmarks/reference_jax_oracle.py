#!/usr/bin/env python
"""Golden trajectories and theory values from the reference's own JAX files, run on NumPy.

    python benchmarks/reference_jax_oracle.py --ref_root <checkout of the reference> [--out FILE]

JAX and Optax are not installed here, but the two files that matter as an oracle use a small part of them:
`jax/optimizers.py` (the second, independent statement of the update rules) needs `jax.numpy`, `jax.tree.map`,
`optax.chain`, `optax.scale_by_learning_rate` and five helpers of `optax._src`; `jax/deterministic_equivalent.py` needs
`jax.numpy` and one `jax.lax.scan`.  This script registers stand-in modules that map those names onto NumPy (float64
unless the reference's code casts, arrays that behave immutably as JAX's do; trees are single arrays or None, which is
all the oracle feeds in), imports the reference's files unmodified, drives
every optimizer factory over a fixed gradient sequence and evaluates the theory functions at fixed arguments, and
writes `tests/golden/theory_reference_values.json` for `tests/test_theory_vs_reference_jax.py`.
"""
import argparse
import importlib.util
import json
import sys
import types
from collections import namedtuple
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent


class JArray(np.ndarray):
    """JAX arrays are immutable: `F = m; F += x` binds a new array to F and leaves m alone, where NumPy would add into
    m.  Arrays made through the stand-in `jax.numpy` are of this subclass, whose in-place operators work out of place;
    ufuncs keep the subclass, so everything derived from them behaves the same way."""

    def __iadd__(self, o):
        return self + o

    def __isub__(self, o):
        return self - o

    def __imul__(self, o):
        return self * o

    def __itruediv__(self, o):
        return self / o

    def __ipow__(self, o):
        return self ** o


def _j(x):
    return x.view(JArray) if isinstance(x, np.ndarray) and not isinstance(x, JArray) else x


def _wrap(fn):
    def wrapped(*a, **k):
        out = fn(*a, **k)
        if isinstance(out, (list, tuple)):
            return type(out)(_j(o) for o in out)
        return _j(out)

    return wrapped


def install_shims():
    jnp = types.ModuleType("jax.numpy")
    jnp.__dict__.update({k: getattr(np, k) for k in dir(np) if not k.startswith("__")})
    jnp.pow = np.power
    for name in ("array", "asarray", "ones", "zeros", "ones_like", "zeros_like", "arange", "linspace", "logspace", "geomspace",
                 "reshape", "split", "concatenate", "outer", "sum", "where", "maximum", "minimum", "exp", "log", "sqrt",
                 "abs", "power", "imag", "real", "cumsum", "trapezoid", "interp", "einsum", "eye", "full", "full_like", "copy"):
        if hasattr(np, name):
            setattr(jnp, name, _wrap(getattr(np, name)))
    for name in ("complex64", "complex128", "float32", "float64", "int32"):     # used both as dtypes and as casts
        t = getattr(np, name)

        def make(tt):      # `dtype=jnp.complex64` still works (NumPy reads the `.dtype` attribute); `jnp.complex64(x)` casts
            class Caster:
                dtype = np.dtype(tt)

                def __call__(self, x):
                    return _j(np.asarray(x, dtype=tt)) if np.ndim(x) else tt(x)

                def __repr__(self):
                    return f"shim.{tt.__name__}"

            return Caster()

        setattr(jnp, name, make(t))

    def tree_map(fn, *trees, is_leaf=None):
        first = trees[0]
        if isinstance(first, dict):
            return {k: tree_map(fn, *[t[k] for t in trees], is_leaf=is_leaf) for k in first}
        if isinstance(first, (list, tuple)) and not hasattr(first, "_fields"):
            return type(first)(tree_map(fn, *ts, is_leaf=is_leaf) for ts in zip(*trees))
        return fn(*trees)

    def scan(f, init, xs):
        carry, ys = init, []
        for x in xs:
            carry, y = f(carry, x)
            ys.append(y)
        if not ys or ys[0] is None:
            return carry, None
        if isinstance(ys[0], tuple):      # a tuple of outputs per step becomes a tuple of stacked arrays
            return carry, tuple(_j(np.stack([np.asarray(y[k]) for y in ys])) for k in range(len(ys[0])))
        return carry, _j(np.stack([np.asarray(y) for y in ys]))

    jax = types.ModuleType("jax")
    jax.numpy = jnp
    jax.tree = types.SimpleNamespace(map=tree_map)
    jax.tree_util = types.SimpleNamespace(tree_map=tree_map)
    jax.lax = types.SimpleNamespace(scan=scan)
    jax.jit = lambda f=None, **kw: f if f is not None else (lambda g: g)

    chex = types.ModuleType("chex")
    for name in ("Scalar", "Array", "ArrayDType", "Numeric", "ArrayTree"):
        setattr(chex, name, object)

    GradientTransformation = namedtuple("GradientTransformation", ["init", "update"])
    base = types.ModuleType("optax._src.base")
    base.GradientTransformation = GradientTransformation
    for name in ("Schedule", "ScalarOrSchedule", "Updates", "Params"):
        setattr(base, name, object)
    numerics = types.ModuleType("optax._src.numerics")
    numerics.safe_increment = lambda c: c + 1
    utils = types.ModuleType("optax._src.utils")
    utils.canonicalize_dtype = lambda d: d
    otu = types.ModuleType("optax.tree_utils")
    otu.tree_zeros_like = lambda tree, dtype=None: tree_map(lambda p: None if p is None else np.zeros_like(p, dtype=dtype), tree)
    otu.tree_cast = lambda tree, dtype=None: tree_map(lambda p: p if (p is None or dtype is None) else np.asarray(p, dtype=dtype), tree)

    def chain(*ts):
        def init(params):
            return tuple(t.init(params) for t in ts)

        def update(updates, state, params=None):
            new = []
            for t, s in zip(ts, state):
                updates, s = t.update(updates, s, params)
                new.append(s)
            return updates, tuple(new)

        return GradientTransformation(init, update)

    def scale_by_learning_rate(lr, flip_sign=True):
        sign = -1.0 if flip_sign else 1.0

        def init(params):
            return np.zeros([], np.int64)

        def update(updates, count, params=None):
            step = lr(count) if callable(lr) else lr
            return tree_map(lambda u: sign * step * u, updates), count + 1

        return GradientTransformation(init, update)

    def adam(learning_rate, b1=0.9, b2=0.999, eps=1e-8):
        def init(params):
            return (0, np.zeros_like(params), np.zeros_like(params))

        def update(g, state, params=None):
            c, m, v = state
            c += 1
            m = b1 * m + (1 - b1) * g
            v = b2 * v + (1 - b2) * g * g
            lr = learning_rate(c - 1) if callable(learning_rate) else learning_rate
            return -lr * (m / (1 - b1 ** c)) / (np.sqrt(v / (1 - b2 ** c)) + eps), (c, m, v)

        return GradientTransformation(init, update)

    def adagrad(learning_rate, initial_accumulator_value=0.1, eps=1e-7):
        def init(params):
            return tree_map(lambda p: np.full_like(np.asarray(p, dtype=np.float64), initial_accumulator_value), params)

        def update(g, acc, params=None):
            acc = tree_map(lambda a, x: a + np.asarray(x) ** 2, acc, g)
            return tree_map(lambda x, a: -learning_rate * np.asarray(x) / (np.sqrt(a) + eps), g, acc), acc

        return GradientTransformation(init, update)

    def apply_updates(params, updates):
        return tree_map(lambda p, u: _j(np.asarray(p) + np.asarray(u)), params, updates)

    def grad(fn, argnums=0):
        """Central differences in place of automatic differentiation (the fits have three to five parameters)."""
        def g(*args):
            x = np.array(args[argnums], dtype=np.float64)
            out = np.zeros_like(x)
            flat, of = x.reshape(-1), out.reshape(-1)
            for i in range(flat.size):
                h = 1e-6 * max(1.0, abs(flat[i]))
                hi, lo = flat.copy(), flat.copy()
                hi[i] += h
                lo[i] -= h
                a_hi = list(args); a_hi[argnums] = _j(hi.reshape(x.shape)) if x.ndim else float(hi[0])
                a_lo = list(args); a_lo[argnums] = _j(lo.reshape(x.shape)) if x.ndim else float(lo[0])
                of[i] = (float(fn(*a_hi)) - float(fn(*a_lo))) / (2 * h)
            return _j(out) if x.ndim else float(out)

        return g

    jax.grad = grad
    optax = types.ModuleType("optax")
    optax.adam, optax.adagrad, optax.apply_updates = adam, adagrad, apply_updates
    optax.chain, optax.scale_by_learning_rate, optax.tree_utils = chain, scale_by_learning_rate, otu
    optax.GradientTransformation = GradientTransformation
    src = types.ModuleType("optax._src")
    src.base, src.numerics, src.utils = base, numerics, utils
    optax._src = src
    jax.random = types.ModuleType("jax.random")          # a key is a NumPy seed here: enough for the constructors' sketch
    jax.random.PRNGKey = lambda seed: int(seed)
    jax.random.normal = lambda key, shape=(), dtype=None: _j(np.random.default_rng(key).standard_normal(shape))
    jax.random.split = lambda key, num=2: [int(key) * 1000 + i + 1 for i in range(num)]

    def categorical(key, logits, shape=()):
        p = np.exp(np.asarray(logits, dtype=np.float64))
        return _j(np.random.default_rng(key).choice(len(p), size=shape, p=p / p.sum()))

    jax.random.categorical = categorical

    def softmax(x, axis=-1):
        z = np.asarray(x) - np.max(x, axis=axis, keepdims=True)
        e = np.exp(z)
        return _j(e / e.sum(axis=axis, keepdims=True))

    jax.nn = types.SimpleNamespace(softmax=softmax, one_hot=lambda idx, n: _j(np.eye(n)[np.asarray(idx)]),
                                   sigmoid=lambda x: 1.0 / (1.0 + np.exp(-x)))
    sys.modules["jax.random"] = jax.random
    sys.modules.update({"jax": jax, "jax.numpy": jnp, "chex": chex, "optax": optax, "optax.tree_utils": otu,
                        "optax._src": src, "optax._src.base": base, "optax._src.numerics": numerics, "optax._src.utils": utils})


def load(path: Path, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def cut_functions(path: Path, names, extra=None):
    """The named top-level functions of a file that cannot be imported (matplotlib at module level), compiled into a
    namespace that holds the stand-in `jax` / `jnp` and typing names."""
    import ast
    from typing import Callable, Literal, NamedTuple, Optional, Union

    tree = ast.parse(path.read_text())
    keep = [n for n in tree.body if isinstance(n, (ast.FunctionDef, ast.ClassDef)) and n.name in names]
    assert {n.name for n in keep} == set(names), (path.name, names)
    ns = {"jax": sys.modules["jax"], "jnp": sys.modules["jax.numpy"], "NamedTuple": NamedTuple, "Callable": Callable, "Union": Union,
          "Optional": Optional, "Literal": Literal}
    ns.update(extra or {})
    for node in keep:                      # annotations name classes of the file that are not taken along
        if isinstance(node, ast.FunctionDef):
            node.returns = None
            for arg in node.args.args + node.args.kwonlyargs:
                arg.annotation = None
    exec(compile(ast.Module(keep, []), str(path), "exec"), ns)
    return ns


def plain(o):
    if isinstance(o, dict):
        return {str(k): plain(v) for k, v in o.items()}
    if isinstance(o, (list, tuple)):
        return [plain(v) for v in o]
    if isinstance(o, np.ndarray):
        if np.iscomplexobj(o):
            return {"re": o.real.tolist(), "im": o.imag.tolist()}
        return o.tolist()
    if isinstance(o, (np.floating, np.integer)):
        return o.item()
    if isinstance(o, complex):
        return {"re": o.real, "im": o.imag}
    return o


def trajectory(opt, grads, p0):
    """Parameters after every step of `p <- p + update` under the reference's gradient transformation."""
    p = _j(np.array(p0, dtype=np.float64))
    state = opt.init(p)
    out = []
    for g in grads:
        upd, state = opt.update(_j(np.array(g, dtype=np.float64)), state, p)
        p = p + upd
        out.append(np.array(p))
    return np.array(out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref_root", required=True)
    ap.add_argument("--out", default=str(ROOT / "tests" / "golden" / "theory_reference_values.json"))
    a = ap.parse_args()
    install_shims()
    jdir = Path(a.ref_root) / "jax"
    O = load(jdir / "optimizers.py", "ref_jax_optimizers")
    D = load(jdir / "deterministic_equivalent.py", "ref_jax_deterministic")
    G = {}

    # ---- update rules: a fixed, partly sparse gradient sequence --------------------------------------------------------
    rng = np.random.default_rng(0)
    steps, n = 40, 6
    grads = rng.standard_normal((steps, n)) * (rng.random((steps, n)) < 0.7) * np.array([1.0, 0.1, 3.0, 1.0, 0.01, 1.0])
    p0 = rng.standard_normal(n)
    lr = lambda c: 0.5 / (1.0 + c / 20.0)
    G["rules"] = {"grads": grads.tolist(), "p0": p0.tolist(), "lr": "0.5 / (1 + count / 20)", "runs": {}}
    cases = {
        "adana_k1": (O.get_adana, dict(g2_constant=0.02, g3_constant=0.01, kappa=1.0, delta=8.0)),
        "adana_k0.8": (O.get_adana, dict(g2_constant=0.02, g3_constant=0.01, kappa=0.8, delta=6.0)),
        "dana_mk4_k0.85": (O.get_dana_mk4, dict(g2_constant=0.02, g3_constant=0.03, kappa=0.85, clipsnr=0.5, delta=8.0)),
        "dana_star_mk4_k0.85": (O.get_dana_star_mk4, dict(g2_constant=0.02, g3_constant=0.03, kappa=0.85, clipsnr=2.0, delta=8.0)),
        "dana_star_mk4_k0.6_tightclip": (O.get_dana_star_mk4, dict(g2_constant=0.05, g3_constant=0.05, kappa=0.6, clipsnr=0.25, delta=4.0)),
    }
    for name, (factory, kw) in cases.items():
        G["rules"]["runs"][name] = {"kwargs": kw, "params": plain(trajectory(factory(learning_rate=lr, **kw), grads, p0))}
    G["rules"]["runs"]["dana_star_k0.7"] = {"kwargs": dict(g2_constant=0.02, g3_constant=0.01, kappa_exponent=0.7),
                                          "params": plain(trajectory(O.get_dana_star(0.02, 0.01, 0.7, lr), grads, p0))}
    beta3 = lambda c: 1.0 - 0.1 / (1.0 + c / 10.0)
    alpha = lambda c: min(c / 20.0, 1.0) * 3.0
    G["rules"]["runs"]["ademamix"] = {"kwargs": dict(beta1=0.9, beta2=0.99, beta3="1 - 0.1 / (1 + count / 10)", alpha="min(count / 20, 1) * 3",
                                                     gamma_3_factor=0.7, weight_decay=0.01),
                                      "params": plain(trajectory(O.get_ademamix(lr, 0.9, 0.99, beta3, alpha, 0.7, 1e-8, 0.01), grads, p0))}
    sched = O.powerlaw_schedule(2.0, 0.05, -0.75, 10.0)
    G["powerlaw_schedule"] = {"args": [2.0, 0.05, -0.75, 10.0], "t": [0, 1, 10, 100, 1e4, 1e6], "values": [float(sched(t)) for t in (0, 1, 10, 100, 1e4, 1e6)]}

    # ---- deterministic equivalent -------------------------------------------------------------------------------------------
    T = {}
    T["limit_loss"] = [{"args": args, "value": float(D.theory_limit_loss(*args))} for args in ((1.0, 0.5, 2000, 200), (0.3, 0.4, 1000, 100), (1.5, 0.3, 2500, 500))]
    T["kappa"] = [{"args": args, "value": float(D.theory_kappa(*args))} for args in ((1.0, 2000, 200), (0.7, 1000, 250))]
    T["tau"] = [{"args": args, "value": float(D.theory_tau(*args))} for args in ((0.3, 2000, 200), (0.45, 1000, 100))]
    T["lambda_min"] = [{"args": args, "value": float(D.theory_lambda_min(*args))} for args in ((1.0, 2000, 200), (0.6, 800, 100))]
    T["rhos"] = [{"args": args, "eigs": plain(np.asarray(D.theory_rhos(*args)[0])), "rho": plain(np.asarray(D.theory_rhos(*args)[1]))}
                 for args in ((1.0, 0.3, 12), (0.8, 0.7, 10))]
    xs = np.geomspace(2e-4, 0.9, 16)
    T["m"] = {"args": dict(v=300, d=60, alpha=1.0), "xs": xs.tolist(), "value": plain(np.asarray(D.theory_m_batched(300, 60, 1.0, xs)))}
    T["f_measure"] = {"args": dict(v=300, d=60, alpha=1.0, beta=0.4), "xs": xs.tolist(),
                      "value": plain(np.asarray(D.theory_f_measure(300, 60, 1.0, 0.4, xs)))}
    T["empirical_measure"] = {"args": dict(v=300, d=60, alpha=1.0), "xs": xs.tolist(),
                              "value": plain(np.asarray(D.theory_empirical_measure(300, 60, 1.0, xs)))}
    dens = np.linspace(0.5, 2.0, 50)
    grid = np.linspace(0.0, 1.0, 50)
    T["chunk_weights"] = {"xs": grid.tolist(), "density": dens.tolist(), "a": [0.0, 0.2, 0.5], "b": [0.2, 0.5, 1.0],
                          "value": plain(np.asarray(D.chunk_weights(grid, dens, np.array([0.0, 0.2, 0.5]), np.array([0.2, 0.5, 1.0]))))}
    spec = np.asarray(D.deterministic_spectra(200, 40, 1.0), dtype=np.float64)
    T["spectra"] = {"args": dict(v=200, d=40, alpha=1.0), "value": spec.tolist()}
    lam = np.arange(1, 13, dtype=np.float64) ** -2.0
    lo, hi = lam * 0.93, lam * 1.07
    T["rho_weights"] = {"args": dict(v=200, d=40, alpha=1.0, beta=0.3), "a": lo.tolist(), "b": hi.tolist(),
                        "value": plain(np.asarray(D.deterministic_rho_weights(200, 40, 1.0, 0.3, _j(lo), _j(hi)), dtype=np.float64))}
    G["deterministic"] = T

    # ---- the risk ODE: the solver of dana_plrf.py and the momentum-tracking variants of the schedule scripts -------------------
    d = 40
    eigs, rho = np.asarray(D.theory_rhos(0.8, 0.4, d)[0], dtype=np.float64), np.asarray(D.theory_rhos(0.8, 0.4, d)[1], dtype=np.float64)
    r_inf = float(D.theory_limit_loss(0.8, 0.4, 4 * d, d))
    ns = cut_functions(jdir / "dana_plrf.py", ["DanaHparams", "ODEInputs", "ode_resolvent_log_implicit"])
    inp = ns["ODEInputs"](_j(eigs), _j(rho), _j(np.zeros(d)), _j(np.zeros(d)), r_inf)
    g1, g2 = (lambda t: 1.0), (lambda t: 0.05)
    g3 = O.powerlaw_schedule(0.02, 0.0, -0.5, 1.0)
    dl = O.powerlaw_schedule(1.0, 0.0, -1.0, 6.0)
    hp = ns["DanaHparams"](g1, g2, g3, dl)
    ode = {"args": dict(alpha=0.8, beta=0.4, d=d, v=4 * d, batch=4, t_max=2000.0, dt=0.05), "risk_infinity": r_inf,
           "schedules": "g1 = 1, g2 = 0.05, g3 = 0.02 (1+t)^-0.5, delta = (1 + t/6)^-1", "runs": {}}
    for name, kw in (("full", {}), ("approximate", dict(approximate=True)), ("adam", dict(adaptive="adam")),
                     ("rmsprop_dana", dict(adaptive="rmsprop_dana"))):
        t, r = ns["ode_resolvent_log_implicit"](inp, hp, 4, d, 2000.0, 0.05, **kw)
        ode["runs"][name] = {"t": plain(np.asarray(t, dtype=np.float64)), "twice_risk": plain(np.asarray(r, dtype=np.float64))}
    consts = dict(RISK_RENORMALIZED=True, A=0.0, B=0.75, BASE_KAPPA=1.0)
    ks = cut_functions(jdir / "kappa_sweep_plot.py", ["ode_resolvent_log_implicit_and_momentum_dynamic"], consts)
    fn = ks["ode_resolvent_log_implicit_and_momentum_dynamic"]
    hp2 = ns["DanaHparams"](dl, lambda t: 0.01, O.powerlaw_schedule(0.01, 0.0, 0.4, 1.0), dl)
    for name, kw in (("momentum_renormalized", dict(risk_renormalized=True, g3_mode="fixed")),
                     ("momentum_plain", dict(risk_renormalized=False, g3_mode="fixed")),
                     ("momentum_dynamic", dict(risk_renormalized=True, g3_mode="dynamic", power_A=0.0, power_B=0.75, base_kappa=1.0))):
        t, r, m = fn(inp, hp2, 4, d, 2000.0, 0.05, **kw)
        ode["runs"][name] = {"t": plain(np.asarray(t, dtype=np.float64)), "twice_risk": plain(np.asarray(r, dtype=np.float64)),
                             "momentum": plain(np.asarray(m, dtype=np.float64))}
    dyn = cut_functions(jdir / "dynamical_schedule_plot.py", ["ode_resolvent_log_implicit_and_momentum_dynamic"])
    t, r, m = dyn["ode_resolvent_log_implicit_and_momentum_dynamic"](inp, ns["DanaHparams"](g1, g2, lambda t: 0.02, dl), 4, d, 2000.0, 0.05, g3_mode="dynamic")
    ode["runs"]["ratio_rule"] = {"t": plain(np.asarray(t, dtype=np.float64)), "twice_risk": plain(np.asarray(r, dtype=np.float64)),
                                 "momentum": plain(np.asarray(m, dtype=np.float64))}
    G["ode"] = ode

    # ---- the power-law random-features problem with a given sketch ------------------------------------------------------------
    sys.path.insert(0, str(jdir))                     # power_law_rf.py imports deterministic_equivalent by name
    sys.modules["deterministic_equivalent"] = D
    P = load(jdir / "power_law_rf.py", "ref_jax_power_law_rf")
    v, dd = 60, 12
    W = np.random.default_rng(5).standard_normal((v, dd)) / np.sqrt(dd)
    prob = P.PowerLawRF(0.9, 0.4, _j(W))
    ws = np.random.default_rng(6).standard_normal((3, dd))
    G["plrf"] = {"alpha": 0.9, "beta": 0.4, "W": W.tolist(), "w": ws.tolist(),
                 "population_trace": float(prob.population_trace),
                 "risk": [float(prob.get_population_risk(_j(w.reshape(dd, 1)))) for w in ws],
                 "hessian_spectra": plain(np.asarray(prob.get_hessian_spectra(), dtype=np.float64)),
                 "rhos": plain(np.asarray(prob.get_rhos(), dtype=np.float64)),
                 "theory_limit_loss": float(prob.get_theory_limit_loss()),
                 "empirical_limit_loss": float(prob.get_empirical_limit_loss())}
    M = load(jdir / "moe_plrf.py", "ref_jax_moe_plrf")
    moe = M.MixtureOfExpertsPLRF(1.1, 0.2, 50, 10, 5, 0.8, 7)
    two = M.TwoExpertPLRF(1.0, 0.3, 40, 8, 0.7, 9) if hasattr(M, "TwoExpertPLRF") else None
    params = np.random.default_rng(8).standard_normal((10, 5))
    G["moe_plrf"] = {"alpha": 1.1, "beta": 0.2, "m": 5, "zeta": 0.8, "W": plain(np.asarray(moe.W)), "params": params.tolist(),
                     "expert_probs": plain(np.asarray(moe.expert_probs, dtype=np.float64)),
                     "risk": float(moe.population_risk(_j(params))),
                     "per_expert": plain(np.asarray(moe.per_expert_population_risk(_j(params)), dtype=np.float64)),
                     "single_risk": float(moe.population_risk(_j(params[:, 0]))),
                     "optimal_risk": float(moe.optimal_risk())}
    if two is not None:
        G["moe_plrf"]["two_expert_probs"] = plain(np.asarray(two.expert_probs, dtype=np.float64))
    # ---- how the sweep generator wires its optimizers: constants from batch / trace, kappa grid, AdEMAMix warm-ups, Adam ----
    sys.modules["optimizers"], sys.modules["moe_plrf"] = O, M
    H = load(jdir / "hummingbird_generate.py", "ref_jax_hummingbird_generate")
    hb_steps, hb_grads = 30, np.random.default_rng(20).standard_normal((30, 5)) * np.array([1.0, 0.2, 2.0, 0.05, 1.0])
    hb_p0 = np.random.default_rng(21).standard_normal(5)
    base = dict(alpha=1.0, v=400, batch_size=20, g2_scale=0.5, g3_over_g2=0.7, tanea_lr_scalar=0.8, kappa_min=0.0, kappa_max=1.0,
                kappa_step=0.5, clipsnr=1.5, delta=6.0, ademamix_beta1=0.9, ademamix_beta2=0.99, adam_lr=0.2, adam_beta1=0.95, adam_beta2=0.99)
    trace_k = float(H.get_traceK(base["alpha"], base["v"]))
    G["hummingbird_rules"] = {"args": base, "traceK": trace_k, "steps": hb_steps, "grads": hb_grads.tolist(), "p0": hb_p0.tolist(), "runs": {}}
    for opt_name in ("dana-star-mk4", "dana-mk4", "dana-star", "ademamix"):
        opts, kappas = H.create_optimizers(types.SimpleNamespace(optimizer=opt_name, **base), trace_k, hb_steps)
        G["hummingbird_rules"]["runs"][opt_name] = {name: plain(trajectory(o, hb_grads, hb_p0)) for name, o in opts.items()}
    for name in ("matplotlib", "matplotlib.pyplot"):          # imported at module level by the sweep scripts, never called here
        sys.modules.setdefault(name, types.ModuleType(name))
    S = load(jdir / "moe_m_sweeps_mk4.py", "ref_jax_moe_m_sweeps_mk4")
    ms = dict(alpha=1.0, beta=0.0, d=50, batch_size=20, g2_scale=0.2, g3_over_g2=0.01, tanea_lr_scalar=1.0, adam_lr=0.2)
    tk = float(S.get_traceK(ms["alpha"], 400))
    common = (ms["alpha"], ms["beta"], ms["d"], ms["batch_size"], ms["g2_scale"], ms["g3_over_g2"], tk, ms["tanea_lr_scalar"], 0.0)
    G["m_sweep_rules"] = {"args": ms, "v": 400, "traceK": tk, "grads": hb_grads.tolist(), "p0": hb_p0.tolist(), "runs": {
        "dana-star": plain(trajectory(S.get_dana_star_optimizer(*common), hb_grads, hb_p0)),
        "dana-star-mk4": plain(trajectory(S.get_dana_star_mk4_optimizer(*common), hb_grads, hb_p0)),
        "dana-star_kappa0.7": plain(trajectory(S.get_dana_star_optimizer(*common, tanea_kappa=0.7), hb_grads, hb_p0))},
        "adam_lr": float(S.get_adam_lr(*common, ms["adam_lr"]))}
    sys.modules["power_law_rf"], sys.modules["deterministic_equivalent"] = P, D
    B = load(jdir / "plrf_ademamix_behavior.py", "ref_jax_plrf_ademamix_behavior")
    cfg = dict(B.CONFIG, alpha=1.2, beta=0.3, v=200, d=40, steps=3000, batch_size=2, lr_scale=0.5, g2=0.5, g3=0.5, delta=8.0, random_seed=3)
    res, r_inf_b = B.run_ode(cfg)
    keep = slice(None, None, 50)
    G["optimizer_comparison"] = {"cfg": {k: v for k, v in cfg.items() if isinstance(v, (int, float, str))}, "risk_infinity": float(r_inf_b),
                                 "runs": {k: {"t": plain(np.asarray(v["t"], dtype=np.float64)[keep]), "loss": plain(np.asarray(v["loss"], dtype=np.float64)[keep])}
                                          for k, v in res.items()}}
    # ---- the weighted learning-rate law as the reference fits it (Adagrad on the same objective; gradients by differences) ----
    viz = Path(a.ref_root) / "visualization"
    fit = cut_functions(viz / "bighead_lr_scaling.py", ["fit_saturated_power_law_weighted"],
                        {"jit": sys.modules["jax"].jit, "grad": sys.modules["jax"].grad, "optax": sys.modules["optax"],
                         "print": lambda *x, **k: None})
    Ps = np.repeat(np.array([2e6, 1e7, 5e7, 2e8, 1e9]), 3)
    ws = np.tile([3.0, 2.0, 1.0], 5)
    lrs_fit = 12.0 * (4e4 + Ps) ** -0.52 * np.exp(np.random.default_rng(30).normal(0, 0.05, len(Ps)))
    a_f, b_f, d_f = fit["fit_saturated_power_law_weighted"](list(Ps), list(lrs_fit), list(ws), n_steps=5000, learning_rate=0.1)
    G["lr_law_fit"] = {"P": Ps.tolist(), "lr": lrs_fit.tolist(), "w": ws.tolist(), "a": float(a_f), "b": float(b_f), "d": float(d_f)}
    # ---- the joint broken-power-law fit with a shared floor, as the scaling comparison runs it -------------------------------
    jf = cut_functions(viz / "compare_scaling_rules_ep.py", ["broken_power_law", "fit_all_saturated_power_laws_joint"],
                       {"jit": sys.modules["jax"].jit, "grad": sys.modules["jax"].grad, "optax": sys.modules["optax"], "np": np,
                        "args": types.SimpleNamespace(compute_weight=False), "print": lambda *x, **k: None})
    Cs = np.geomspace(0.05, 60, 8)
    law = lambda C, a, b, c, e, f: a + b * C ** -c + e * C ** -f
    data_list = [{"name": "adamw", "compute": Cs, "loss": law(Cs, 1.7, 0.5, 0.30, 1.0, 0.06)},
                 {"name": "dana-star-mk4", "compute": Cs, "loss": law(Cs * 1.5, 1.7, 0.5, 0.30, 1.0, 0.06)}]
    ref_fit = jf["fit_all_saturated_power_laws_joint"]([{**d, "compute": _j(d["compute"]), "loss": _j(d["loss"])} for d in data_list],
                                                       n_steps=20000, learning_rate=0.1)
    G["joint_fit"] = {"curves": [{"name": d["name"], "compute": d["compute"].tolist(), "loss": d["loss"].tolist()} for d in data_list],
                      "reference": plain(ref_fit)}
    L = load(jdir / "lr_plrf.py", "ref_jax_lr_plrf")
    lp = L.LogisticRegressionPLRF(1.0, 0.5, 0.8, 2.0, 30, 8, 5, 11)
    X, Y = lp.generate_batch(21, 64)
    theta = np.random.default_rng(12).standard_normal((8, 5)) * 0.3
    bias = np.random.default_rng(13).standard_normal(5) * 0.1
    G["logistic_plrf"] = {"alpha": 1.0, "beta": 0.5, "zeta": 0.8, "snr": 2.0, "v": 30, "d": 8, "m": 5,
                          "W": plain(np.asarray(lp.W)), "mu": plain(np.asarray(lp.mu)), "class_probs": plain(np.asarray(lp.class_probs, dtype=np.float64)),
                          "sigma_eps_diag": plain(np.asarray(lp.Sigma_eps_diag, dtype=np.float64)),
                          "X": plain(np.asarray(X)), "classes": np.argmax(np.asarray(Y), axis=1).tolist(),
                          "theta": theta.tolist(), "bias": bias.tolist(),
                          "cross_entropy": float(lp.cross_entropy_loss((_j(theta), _j(bias)), X, Y))}
    Path(a.out).write_text(json.dumps(plain(G)))
    print(f"wrote {a.out}")


if __name__ == "__main__":
    main()
