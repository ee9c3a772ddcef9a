"""Power-law random-features regression: the synthetic problem the optimizer theory is stated on.

Hidden dimension v, embedded dimension d, random features W [v, d] ~ N(0, 1/d).  Data x ~ N(0, I_v) are seen
through `x @ (D W)` with D = diag(j^-alpha); the target is `x @ (j^-(alpha+beta))`.  The population risk of
weights w is ||D W w - D b||^2 / 2 with b_j = j^-beta — available in closed form, no sampling needed.
(Reference: jax/power_law_rf.py:8-213; trainer loop: jax/moe_plrf.py:110-210.)
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import numpy as np


class PowerLawRF:
    def __init__(self, alpha: float, beta: float, W: np.ndarray):
        self.alpha, self.beta = alpha, beta
        self.W = np.asarray(W, dtype=np.float64)
        self.v, self.d = self.W.shape
        j = np.arange(1, self.v + 1, dtype=np.float64)
        self.population_eigenvalues = j ** (-alpha)
        self.checkW = self.W * self.population_eigenvalues[:, None]           # D W
        self.checkb = j ** (-(alpha + beta))                                   # D b
        self.population_trace = float(np.sum(self.population_eigenvalues ** 2))

    @classmethod
    def initialize_random(cls, alpha, beta, v, d, seed=0):
        rng = np.random.default_rng(seed)
        return cls(alpha, beta, rng.standard_normal((v, d)) / np.sqrt(d))

    def population_risk(self, w) -> float:
        r = self.checkW @ np.asarray(w, dtype=np.float64).reshape(-1) - self.checkb
        return 0.5 * float(r @ r)

    def hessian_spectrum(self):
        return np.linalg.svd(self.checkW, compute_uv=False) ** 2

    def rhos(self):
        """Squared projections of the target onto the Hessian's eigen-directions, divided by the eigenvalues:
        the initial condition rho_j of the risk ODE for w0 = 0."""
        U, s, _ = np.linalg.svd(self.checkW, full_matrices=False)
        return (self.checkb @ U) ** 2 / s ** 2

    def sample(self, rng: np.random.Generator, batch: int):
        x = rng.standard_normal((batch, self.v))
        return x @ self.checkW, x @ self.checkb

    def batch_gradient(self, w, X, y):
        """Gradient of the batch-averaged half squared error."""
        return X.T @ (X @ w - y) / X.shape[0]

    def limit_risk(self) -> float:
        """Risk of the least-squares solution (what training converges to)."""
        w, *_ = np.linalg.lstsq(self.checkW, self.checkb, rcond=None)
        return self.population_risk(w)


def train_plrf(problem: PowerLawRF, rule, steps: int, batch: int, seed: int = 0,
               eval_at: Optional[Sequence[int]] = None, w0: Optional[np.ndarray] = None,
               on_step: Optional[Callable] = None):
    """One-pass SGD-type training with a `(init, update)` rule; returns (eval steps, population risks, w)."""
    rng = np.random.default_rng(seed)
    w = np.zeros(problem.d) if w0 is None else np.array(w0, dtype=np.float64)
    init, update = rule
    state = init(w)
    if eval_at is None:
        eval_at = np.unique(np.round(np.geomspace(1, steps, 40)).astype(int))
    eval_set = set(int(e) for e in eval_at)
    ts, risks = [0], [problem.population_risk(w)]
    for t in range(1, steps + 1):
        X, y = problem.sample(rng, batch)
        g = problem.batch_gradient(w, X, y)
        dw, state = update(g, state, w)
        w = w + dw
        if on_step is not None:
            on_step(t, w, g, state)
        if t in eval_set:
            ts.append(t)
            risks.append(problem.population_risk(w))
    return np.array(ts), np.array(risks), w
