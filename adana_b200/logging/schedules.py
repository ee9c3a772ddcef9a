"""Scalar logs derived from optimizer state (metric names read by the plotting scripts:
`optimizer/alpha_schedule`, `optimizer/kappa_factor_schedule`, `optimizer/auto_factor`,
`optimizer/g2_gradient_norm`, `optimizer/m_norm`, `optimizer/one_minus_beta3_schedule`).
Behaviour parity: reference src/optim/utils.py:462-615.
"""
from __future__ import annotations

import torch

_KEYS = {"current_alpha": "optimizer/alpha_schedule", "current_kappa_factor": "optimizer/kappa_factor_schedule",
         "auto_factor_mean": "optimizer/auto_factor", "g2_gradient_norm": "optimizer/g2_gradient_norm",
         "m_norm": "optimizer/m_norm", "current_one_minus_beta3": "optimizer/one_minus_beta3_schedule"}


def _as_float(v):
    if isinstance(v, (int, float)):
        return float(v)
    try:
        return float(v.item()) if hasattr(v, "item") else float(v)
    except (RuntimeError, ValueError):
        return None


def get_parameter_norms(model, order=2):
    order = float(order)
    norms = [p.detach().norm(p=order).item() for p in model.parameters() if p.numel()]
    if not norms:
        return 0.0
    if order == float("inf"):
        return max(norms)
    return sum(n ** order for n in norms) ** (1.0 / order)


def log_prodigy_lr(opt):
    out = []
    for g in opt.param_groups:
        bc = 1.0
        if g.get("use_bias_correction"):
            b1, b2 = g["betas"]
            k = g["k"]
            bc = ((1 - b2 ** (k + 1)) ** 0.5) / (1 - b1 ** (k + 1))
        out.append(g["d"] * g["lr"] * bc)
    return out


def log_optimizer_schedules(optimizer, optimizer_name):
    """Mean over parameters of the logged per-parameter scalars."""
    if optimizer_name == "ademamix":  # not the decaying-wd variant, as in the reference (src/optim/utils.py:550)
        wanted = ("current_alpha", "current_one_minus_beta3")
    elif optimizer_name in ("adana", "dana-mk4", "dana-star", "dana-star-mk4"):
        wanted = ("current_alpha", "current_kappa_factor", "auto_factor_mean", "g2_gradient_norm", "m_norm")
    else:
        return {}
    fused = getattr(optimizer, "diagnostics", None)
    if isinstance(fused, dict) and fused:  # the fused engine optimizer reports aggregate values directly
        # (the per-tensor classes have a boolean attribute of the same name)
        return {_KEYS[k]: v for k, v in fused.items() if k in wanted and k in _KEYS}
    acc = {k: [] for k in wanted}
    for group in optimizer.param_groups:
        for p in group["params"]:
            st = optimizer.state.get(p)
            if not st or "current_alpha" not in st:
                continue
            for k in wanted:
                if k in st:
                    v = _as_float(st[k])
                    if v is not None:
                        acc[k].append(v)
    if not acc["current_alpha"]:
        return {}
    return {_KEYS[k]: sum(v) / len(v) for k, v in acc.items() if v}
