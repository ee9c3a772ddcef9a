"""Further synthetic problems of the optimizer theory: mixtures of experts on the power-law random-features
problem, and power-law logistic regression with many classes.  NumPy, CPU.

`MixtureOfExpertsPLRF`   m experts share the random features of a `PowerLawRF` and each has its own weight
    column; a sample is routed to expert i with probability p(i) ~ i^(-zeta), so the rare experts see few
    samples: the setting in which a per-coordinate update clock (the tau estimator of Dana-Star) matters.
    `train_moe_plrf` is the trainer: one routed SGD-type step per iteration with any `(init, update)` rule of
    `theory/rules.py`, population risk per expert and the per-expert update / sample counts
    (reference: jax/moe_plrf.py:212-612).
`LogisticPLRF`   m classes with power-law frequencies p(c) ~ c^(-zeta), class means with covariance
    snr * diag(j^(-2 beta)), noise covariance diag(j^(-2 alpha)), seen through a random d x v map; softmax
    regression with a bias, cross-entropy risk estimated on a fixed evaluation batch
    (reference: jax/lr_plrf.py:22-282, jax/largeclass_logistic.py:35-190 — the two files state the same problem).
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import numpy as np

from .plrf import PowerLawRF


def log_spaced_steps(num_steps: int, ratio: float = 1.1) -> np.ndarray:
    """0 and the integers floor(ratio^k) up to `num_steps` (the reference's default evaluation times)."""
    k = np.arange(1, int(np.ceil(np.log(max(num_steps, 2)) / np.log(ratio))))
    return np.unique(np.concatenate([[0], np.floor(ratio ** k).astype(int), [num_steps]]))


# ---- mixture of experts -------------------------------------------------------------------------------------------
class MixtureOfExpertsPLRF(PowerLawRF):
    def __init__(self, alpha: float, beta: float, W: np.ndarray, m: int, zeta: float,
                 expert_probs: Optional[Sequence[float]] = None):
        super().__init__(alpha, beta, W)
        self.m, self.zeta = int(m), float(zeta)
        p = np.arange(1, self.m + 1, dtype=np.float64) ** (-zeta) if expert_probs is None else np.asarray(expert_probs, float)
        self.expert_probs = p / p.sum()

    @classmethod
    def initialize_random(cls, alpha, beta, v, d, m, zeta, seed=0):
        rng = np.random.default_rng(seed)
        return cls(alpha, beta, rng.standard_normal((v, d)) / np.sqrt(d), m, zeta)

    @classmethod
    def two_experts(cls, alpha, beta, v, d, p, seed=0):
        """Expert 0 with probability 1 - p, expert 1 with probability p (jax/moe_plrf.py:378-408)."""
        rng = np.random.default_rng(seed)
        return cls(alpha, beta, rng.standard_normal((v, d)) / np.sqrt(d), 2, 1.0, expert_probs=[1 - p, p])

    def per_expert_population_risk(self, params: np.ndarray) -> np.ndarray:
        """params [d, m] -> half squared error of every expert's column."""
        r = self.checkW @ params - self.checkb[:, None]
        return 0.5 * np.sum(r * r, axis=0)

    def population_risk(self, params) -> float:
        params = np.asarray(params, dtype=np.float64)
        if params.ndim == 1:
            return super().population_risk(params)
        return float(self.expert_probs @ self.per_expert_population_risk(params))

    def sample_routed(self, rng: np.random.Generator, batch: int):
        X, y = self.sample(rng, batch)
        return X, y, rng.choice(self.m, size=batch, p=self.expert_probs)

    def routed_gradient(self, params: np.ndarray, X, y, experts):
        """Gradient of mean_b 0.5 (x_b . theta_{e_b} - y_b)^2 with respect to params [d, m], and the number of samples
        each expert received."""
        pred = np.einsum("bd,db->b", X, params[:, experts])
        resid = (pred - y) / X.shape[0]
        G = np.zeros_like(params)
        np.add.at(G.T, experts, X * resid[:, None])
        return G, np.bincount(experts, minlength=self.m).astype(np.float64)


def train_moe_plrf(problem: MixtureOfExpertsPLRF, rule, steps: int, batch: int, seed: int = 0,
                   eval_at: Optional[Sequence[int]] = None, init_params: Optional[np.ndarray] = None,
                   track_per_expert: bool = False, track_counts: bool = False) -> Dict[str, np.ndarray]:
    """Routed one-pass training (jax/moe_plrf.py:411-612).  Returns timestamps, losses, final_params, the number of
    steps in which each expert was updated (`expert_update_counts`) and of samples it saw (`expert_sample_counts`);
    optionally the per-expert risks and the count histories at the evaluation times."""
    rng = np.random.default_rng(seed)
    params = np.zeros((problem.d, problem.m)) if init_params is None else np.array(init_params, dtype=np.float64)
    init, update = rule
    state = init(params)
    eval_at = log_spaced_steps(steps) if eval_at is None else np.asarray(eval_at)
    eval_set = set(int(e) for e in eval_at)
    ts, losses = [0], [problem.population_risk(params)]
    per_expert = [problem.per_expert_population_risk(params)]
    upd, seen = np.zeros(problem.m), np.zeros(problem.m)
    hist = {"timestamps": [0], "update_counts": [upd.copy()], "sample_counts": [seen.copy()]}
    for t in range(1, steps + 1):
        X, y, experts = problem.sample_routed(rng, batch)
        G, n_e = problem.routed_gradient(params, X, y, experts)
        d_params, state = update(G, state, params)
        params = params + d_params
        upd += n_e > 0
        seen += n_e
        if t in eval_set:
            ts.append(t)
            losses.append(problem.population_risk(params))
            per_expert.append(problem.per_expert_population_risk(params))
            hist["timestamps"].append(t)
            hist["update_counts"].append(upd.copy())
            hist["sample_counts"].append(seen.copy())
    out = {"timestamps": np.array(ts), "losses": np.array(losses), "final_params": params,
           "expert_update_counts": upd, "expert_sample_counts": seen}
    if track_per_expert:
        out["per_expert_losses"] = np.array(per_expert)
    if track_counts:
        out["update_history"] = {k: np.array(v) for k, v in hist.items()}
    return out


# ---- logistic regression with power-law classes ----------------------------------------------------------------------
class LogisticPLRF:
    def __init__(self, alpha: float, beta: float, zeta: float, snr: float, v: int, d: int, m: int, seed: int = 0,
                 eval_samples: int = 10000):
        rng = np.random.default_rng(seed)
        self.alpha, self.beta, self.zeta, self.snr, self.v, self.d, self.m = alpha, beta, zeta, snr, v, d, m
        self.W = rng.standard_normal((d, v)) / np.sqrt(d)
        p = np.arange(1, m + 1, dtype=np.float64) ** (-zeta)
        self.class_probs = p / p.sum()
        j = np.arange(1, v + 1, dtype=np.float64)
        self.mu = (rng.standard_normal((m, v)) * np.sqrt(snr * j ** (-2.0 * beta))).T      # [v, m]
        self.noise_std = j ** (-alpha)
        # the population risk is estimated on one fixed batch, like the reference's fixed-seed evaluation
        self._eval = self.sample(np.random.default_rng(42), eval_samples)

    def sample(self, rng: np.random.Generator, batch: int):
        c = rng.choice(self.m, size=batch, p=self.class_probs)
        x = rng.standard_normal((batch, self.v)) * self.noise_std + self.mu[:, c].T
        return x @ self.W.T, c

    @staticmethod
    def _log_softmax(logits):
        z = logits - logits.max(axis=1, keepdims=True)
        return z - np.log(np.exp(z).sum(axis=1, keepdims=True))

    def cross_entropy(self, params, X, c) -> float:
        theta, b = params
        return float(-self._log_softmax(X @ theta + b)[np.arange(len(c)), c].mean())

    def population_risk(self, params) -> float:
        return self.cross_entropy(params, *self._eval)

    def gradient(self, params, X, c):
        theta, b = params
        p = np.exp(self._log_softmax(X @ theta + b))
        p[np.arange(len(c)), c] -= 1.0
        p /= X.shape[0]
        return X.T @ p, p.sum(axis=0)


def train_logistic_plrf(problem: LogisticPLRF, rule, steps: int, batch: int, seed: int = 0,
                        eval_at: Optional[Sequence[int]] = None) -> Dict[str, np.ndarray]:
    """Softmax regression (weights [d, m] and a bias [m], both through the same rule) on one pass of samples."""
    rng = np.random.default_rng(seed)
    theta, b = np.zeros((problem.d, problem.m)), np.zeros(problem.m)
    init, update = rule
    s_theta, s_b = init(theta), init(b)
    eval_at = log_spaced_steps(steps) if eval_at is None else np.asarray(eval_at)
    eval_set = set(int(e) for e in eval_at)
    ts, losses = [0], [problem.population_risk((theta, b))]
    for t in range(1, steps + 1):
        X, c = problem.sample(rng, batch)
        g_theta, g_b = problem.gradient((theta, b), X, c)
        d_theta, s_theta = update(g_theta, s_theta, theta)
        d_b, s_b = update(g_b, s_b, b)
        theta, b = theta + d_theta, b + d_b
        if t in eval_set:
            ts.append(t)
            losses.append(problem.population_risk((theta, b)))
    return {"timestamps": np.array(ts), "losses": np.array(losses), "final_params": (theta, b)}
