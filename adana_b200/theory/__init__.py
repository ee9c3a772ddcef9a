"""CPU-side theory tools: a second, independent statement of the log-time optimizer rules (oracle for the
PyTorch classes and the CUDA kernel), the power-law random-features (PLRF) test problem, and the log-time
implicit-Euler solver for its risk dynamics.  NumPy only; nothing here touches a GPU.

Counterpart of the reference's `jax/` package (optimizers.py, power_law_rf.py, dana_plrf.py), which is
written for JAX/Optax; the rules are restated here in NumPy with the convention differences made explicit.
"""
from .ode import DanaHparams, ODEInputs, solve_risk_ode  # noqa: F401
from .plrf import PowerLawRF, train_plrf  # noqa: F401
from .sweeps import compare_rules, final_risk_exponent, sweep, tau_order_statistics  # noqa: F401
from .rules import (ademamix_rule, adana_rule, dana_mk4_rule, dana_star_mk4_rule, powerlaw_schedule,  # noqa: F401
                    scale_by_learning_rate)
