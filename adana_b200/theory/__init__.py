"""CPU-side theory tools: a second, independent statement of the log-time optimizer rules (oracle for the
PyTorch classes and the CUDA kernel), the power-law random-features (PLRF) test problem, and the log-time
implicit-Euler solver for its risk dynamics.  NumPy only; nothing here touches a GPU.

Counterpart of the reference's `jax/` package, which is written for JAX/Optax; restated here in NumPy with the
convention differences made explicit: `rules.py` (optimizers.py), `plrf.py` (power_law_rf.py), `ode.py` (dana_plrf.py),
`deterministic.py` (deterministic_equivalent.py: limit loss, kappa, tau, smallest eigenvalue, the fixed point m(z),
spectral densities and rho weights by contour integrals), `problems.py` (moe_plrf.py, lr_plrf.py,
largeclass_logistic.py: mixture-of-experts and power-law logistic problems with their trainers), `generate.py`
(hummingbird_generate.py, taustats_generate.py: the sweep generators; figures are drawn by `adana_b200.figures`).
"""
from .ode import DanaHparams, ODEInputs, solve_risk_ode  # noqa: F401
from .plrf import PowerLawRF, train_plrf  # noqa: F401
from .sweeps import compare_rules, final_risk_exponent, sweep, tau_order_statistics  # noqa: F401
from .rules import (ademamix_rule, adana_rule, dana_mk4_rule, dana_star_mk4_rule, dana_star_rule, powerlaw_schedule,  # noqa: F401
                    scale_by_learning_rate)
from .deterministic import (deterministic_rho_weights, deterministic_spectra, spectral_density, theory_empirical_measure,  # noqa: F401
                            theory_f_measure, theory_kappa, theory_lambda_min, theory_limit_loss, theory_m, theory_rhos,
                            theory_tau)
from .problems import (LogisticPLRF, MixtureOfExpertsPLRF, log_spaced_steps, train_logistic_plrf,  # noqa: F401
                       train_moe_plrf)
