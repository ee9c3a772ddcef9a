"""Deterministic equivalent of the power-law random-features (PLRF) problem: closed forms and spectral densities.

For features with population spectrum lambda_j = j^(-2 alpha), j = 1..v, seen through a random d-dimensional
sketch, the sketched covariance has a deterministic limit described by the fixed point

    m(z) + (1/d) sum_j lambda_j m(z) / (lambda_j m(z) - z) = 1,

from which follow the risk at time infinity, the smallest eigenvalue, the spectral density and the weights
rho_j with which the target (coefficients j^(-beta)) loads on each eigen-direction; those weights and the
eigenvalues are what the log-time risk ODE (`theory/ode.py`) integrates.  NumPy / SciPy restatement of the
quantities the reference computes with JAX in jax/deterministic_equivalent.py:7-551 (same definitions, so its
figures can be regenerated from these functions); risk is MSE / 2 throughout.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import numpy as np


# ---- scalar closed forms ------------------------------------------------------------------------------------------
def theory_kappa(alpha: float, V: int, D: int, tol: float = 1e-3) -> float:
    """Self-consistent kappa for 2 alpha >= 1: kappa = 1 / int_0^{V/D} dx / (kappa + x^(2 alpha)), started from the
    V/D -> infinity value (jax/deterministic_equivalent.py:36-61)."""
    from scipy.integrate import quad

    c, _ = quad(lambda x: 1.0 / (1.0 + x ** (2 * alpha)), 0.0, 1000.0)
    kappa = c ** (-2.0 * alpha)
    for _ in range(10_000):
        nxt = 1.0 / quad(lambda x: 1.0 / (kappa + x ** (2 * alpha)), 0.0, V / D)[0]
        done = abs(nxt / kappa - 1.0) <= tol
        kappa = nxt
        if done:
            break
    return float(kappa)


def theory_tau(alpha: float, V: int, D: int, tol: float = 1e-3) -> float:
    """Self-consistent tau for 2 alpha < 1: tau = 1 / sum_{j<V} 1 / (D (j^(2 alpha) + tau)) (:64-86)."""
    j = np.arange(1, V, dtype=np.float64) ** (2 * alpha)
    it = lambda k: float(np.sum(1.0 / (D * (j + k))))
    tau = it(0.0)
    for _ in range(10_000):
        nxt = 1.0 / it(tau)
        done = abs(nxt / tau - 1.0) <= tol
        tau = nxt
        if done:
            break
    return float(tau)


def theory_limit_loss(alpha: float, beta: float, V: int, D: int) -> float:
    """Risk at time infinity with finite V, D corrections (assumes V > D) (:7-32)."""
    j = np.arange(1, V, dtype=np.float64)
    num = j ** (-2.0 * (beta + alpha))
    if 2 * alpha >= 1.0:
        c = np.sum(num / (j ** (-2.0 * alpha) * theory_kappa(alpha, V, D) * D ** (2 * alpha) + 1.0))
    else:
        c = np.sum(num / (j ** (-2.0 * alpha) * theory_tau(alpha, V, D) + 1.0))
    return float(c) / 2.0


def theory_lambda_min(alpha: float, V: int, D: int, iters: int = 100, tol: float = 1e-10) -> float:
    """Smallest eigenvalue of the deterministic equivalent: bisect 1 = (1/D) sum_j lambda_j^2 u^2 / (lambda_j u - 1)^2
    for u in [-(V/D) kappa D^(2 alpha), 0], then z = 1/u - (1/D) sum_j lambda_j / (lambda_j u - 1) (:88-151)."""
    lam = np.arange(1, V + 1, dtype=np.float64) ** (-2.0 * alpha)
    a, b = -(V / D) * theory_kappa(alpha, V, D) * D ** (2 * alpha), 0.0
    u = 0.5 * (a + b)
    for _ in range(iters):
        u = 0.5 * (a + b)
        f = 1.0 - np.sum(lam ** 2 * u ** 2 / (lam * u - 1.0) ** 2) / D
        if abs(f) < tol:
            break
        if f > 0:
            b = u
        else:
            a = u
    return float(1.0 / u - np.sum(lam / (lam * u - 1.0)) / D)


def theory_rhos(alpha: float, beta: float, d: int) -> Tuple[np.ndarray, np.ndarray]:
    """Leading-order eigenvalues j^(-2 alpha) and weights: the pure-point part j^(-2 beta) plus, for alpha, beta > 1/2,
    the flat part sum_j j^(-2 beta) / d (:154-177)."""
    j = np.arange(1, d + 1, dtype=np.float64)
    flat = np.sum(j ** (-2.0 * beta)) / d if (beta > 0.5 and alpha > 0.5) else 0.0
    return j ** (-2.0 * alpha), j ** (-2.0 * beta) + flat


# ---- the fixed point m(z) -----------------------------------------------------------------------------------------
def theory_m(v: int, d: int, alpha: float, xs: np.ndarray, eta: float = -6.0, eta0: float = 6.0, eta_steps: int = 50,
             x_batch: int = 1000) -> np.ndarray:
    """m(x + i 10^eta) by Newton's method with continuation in the imaginary part: start far from the axis
    (10^eta0, where m = 1 is a good guess) and walk down a logarithmic ladder, one Newton step per rung, carrying the
    solution along (:180-259).  `xs` may be complex (the real axis offset)."""
    xs = np.asarray(xs, dtype=np.complex128)
    lam = np.arange(1, v + 1, dtype=np.float64) ** (-2.0 * alpha)
    etas = np.logspace(eta0, eta, num=int(eta_steps))
    out = np.empty_like(xs)
    for s in range(0, len(xs), x_batch):
        x = xs[s:s + x_batch]
        m = np.ones_like(x)
        for e in etas:
            z = x + 1j * e
            lm = lam[:, None] * m[None, :]
            den = lm - z[None, :]
            F = m + (lm / den).sum(0) / d - 1.0
            Fp = 1.0 - (lam[:, None] * z[None, :] / den ** 2).sum(0) / d
            m = m - F / Fp
        out[s:s + x_batch] = m
    return out


def _newton_ladder(d: int, alpha: float, err: float):
    eps = 10.0 ** err
    eta = float(np.log10(eps * d ** (-2 * alpha)))
    steps = int(40 + 10 * (2 * alpha) * np.log(d))
    return eps, eta, steps


def theory_f_measure(v: int, d: int, alpha: float, beta: float, xs: np.ndarray, err: float = -6.0,
                     m_fn: Optional[Callable] = None) -> np.ndarray:
    """Density of the target-weighted spectral measure biased by 1/z: Im[ sum_j j^(-2(alpha+beta)) / (lambda_j m - z) / z ]
    / pi on the points xs (what the rho_j weights integrate) (:262-321)."""
    xs = np.asarray(xs)
    eps, eta, steps = _newton_ladder(d, alpha, err)
    zs = xs + 1j * eps
    ms = (m_fn or theory_m)(v, d, alpha, zs, eta, 6.0, steps)
    j = np.arange(1, v + 1, dtype=np.float64)
    lam, w = j ** (-2.0 * alpha), j ** (-2.0 * (alpha + beta))
    F = (w[:, None] / (lam[:, None] * ms[None, :] - (zs + 1j * 10.0 ** eta)[None, :])).sum(0)
    return np.imag(F / zs) / np.pi


def theory_empirical_measure(v: int, d: int, alpha: float, xs: np.ndarray, err: float = -6.0,
                             m_fn: Optional[Callable] = None) -> np.ndarray:
    """Density of the eigenvalues of the deterministic equivalent itself (unit weights) (:432-489)."""
    xs = np.asarray(xs)
    eps, eta, steps = _newton_ladder(d, alpha, err)
    zs = xs + 1j * eps
    ms = (m_fn or theory_m)(v, d, alpha, zs, eta, 6.0, steps)
    lam = np.arange(1, v + 1, dtype=np.float64) ** (-2.0 * alpha)
    E = (1.0 / (lam[:, None] * ms[None, :] - (zs + 1j * 10.0 ** eta)[None, :])).sum(0)
    return np.imag(E) / np.pi


def chunk_weights(xs: np.ndarray, density: np.ndarray, a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Riemann sums of `density` (on the uniform grid xs) over the intervals [a_i, b_i] (:324-341)."""
    dx = xs[1] - xs[0]
    return np.array([float(np.sum(density[(xs >= lo) & (xs <= hi)]) * dx) for lo, hi in zip(a, b)])


def deterministic_rho_weights(v: int, d: int, alpha: float, beta: float, a: np.ndarray, b: np.ndarray,
                              xs_per_split: Optional[int] = None, f_measure_fn: Callable = theory_f_measure) -> np.ndarray:
    """rho_j weights as many small contour integrals, one per interval [a_i, b_i] around an eigenvalue, returned from
    the largest eigenvalue to the smallest.  The axis is cut into geometrically shrinking bins (ratio 1 - 1/sqrt(j+2));
    every bin that holds intervals gets its own uniform grid of `xs_per_split` points (default d) (:344-429)."""
    xs_per_split = int(xs_per_split or d)
    order = np.argsort(-np.asarray(a))
    a, b = np.asarray(a, dtype=np.float64)[order], np.asarray(b, dtype=np.float64)[order]
    weights = []
    for lo, hi in _shrinking_bins(a.min() * 0.5):
        idx = np.where((a >= lo) & (a <= hi))[0]
        if len(idx) == 0:
            continue
        xs = np.linspace(a[idx].min(), b[idx].max(), xs_per_split)
        density = f_measure_fn(v, d, alpha, beta, xs, err=-20.0)
        weights.append(chunk_weights(xs, density, a[idx], b[idx]))
    out = np.concatenate(weights) if weights else np.array([])
    if len(out) != len(a):
        raise ValueError(f"generated {len(out)} weights for {len(a)} intervals (an interval fell outside every bin)")
    return out


def _shrinking_bins(left_edge: float, right_edge: float = 2.2):
    """(left, right) ends of the bins that cut [left_edge, right_edge] from the right with ratios 1 - 1/sqrt(j + 2)."""
    seq, cur, j = [], right_edge, 1.0
    while cur >= left_edge:
        seq.append(cur)
        cur *= 1.0 - 1.0 / np.sqrt(j + 2.0)
        j += 1.0
    return list(zip(seq[1:], seq[:-1]))


def spectral_density(v: int, d: int, alpha: float, points: Optional[int] = None) -> Tuple[np.ndarray, np.ndarray]:
    """(grid, density) of the eigenvalue distribution of the deterministic equivalent between half its smallest
    eigenvalue and just above the largest population eigenvalue, on one geometric grid (for drawing)."""
    n = int(points or 10 * d)
    lo = max(theory_lambda_min(alpha, v, d) * 0.5, 1e-12)
    xs = np.geomspace(lo, 1.1, n)
    return xs, theory_empirical_measure(v, d, alpha, xs)


def deterministic_spectra(v: int, d: int, alpha: float, xs_per_split: Optional[int] = None) -> np.ndarray:
    """Eigenvalues of the deterministic equivalent, largest first: the points where the (unnormalised) distribution
    function of its spectral measure, accumulated from the right over shrinking bins with `xs_per_split` grid points
    each (default d), crosses a half-integer (:492-551)."""
    n = int(xs_per_split or d)
    spectra, carried = [], 0.0
    for left, right in _shrinking_bins(theory_lambda_min(alpha, v, d) * 0.5):
        xs = np.linspace(left, right, n)
        density = theory_empirical_measure(v, d, alpha, xs, err=-20.0)
        cdf = np.cumsum(density) * (xs[1] - xs[0])
        cdf = (cdf[-1] + carried) - cdf            # mass to the right of each grid point
        carried = cdf[0]
        frac = cdf - np.floor(cdf)
        hit = (cdf[:-1] > cdf[1:]) & (frac[:-1] > 0.5) & (frac[1:] < 0.5)
        spectra.extend(xs[:-1][hit].tolist())
    return np.sort(np.array(spectra))[::-1]
