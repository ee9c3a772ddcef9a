"""Scaling rules: model shape and peak learning rate from a head count.

`--scaling_rule enoki --heads h` gives L = 3h//4, d = 64h, mlp = 4d, head_dim 64;
`qwen3` gives L = 2h, d = 128h, mlp = 3d, head_dim 128.  The peak LR follows a saturated
power law of the non-embedding parameter count, with per-optimizer (and per-kappa) fits
and a separate table for global batch 512.  Behaviour parity: reference
src/config/scaling.py:19-160.  Shape formulas are small arithmetic expressions evaluated
by a whitelisting AST walker (no `eval`).
"""
from __future__ import annotations

import ast
import operator
from functools import lru_cache
from pathlib import Path

import yaml

_OPS = {ast.Add: operator.add, ast.Sub: operator.sub, ast.Mult: operator.mul,
        ast.FloorDiv: operator.floordiv, ast.Div: operator.truediv, ast.Pow: operator.pow}


def _arith(expr: str, env: dict) -> int:
    def ev(n):
        if isinstance(n, ast.Expression):
            return ev(n.body)
        if isinstance(n, ast.Constant) and isinstance(n.value, (int, float)):
            return n.value
        if isinstance(n, ast.Name) and n.id in env:
            return env[n.id]
        if isinstance(n, ast.BinOp) and type(n.op) in _OPS:
            return _OPS[type(n.op)](ev(n.left), ev(n.right))
        raise ValueError(f"unsupported term in scaling formula {expr!r}")
    return ev(ast.parse(expr, mode="eval"))


@lru_cache(maxsize=1)
def load_rules() -> dict:
    with open(Path(__file__).with_name("scaling_rules.yaml")) as f:
        return yaml.safe_load(f)


def compute_dimensions(rule_name: str, heads: int) -> dict:
    table = load_rules()
    rules = table["rules"]
    if rule_name not in rules:
        raise ValueError(f"Unknown scaling rule: '{rule_name}'. Available: {sorted(rules)}")
    r = rules[rule_name]
    width = int(_arith(r["width"], {"heads": heads}))
    layers = int(_arith(r["layers"], {"heads": heads}))
    mlp = int(_arith(r["mlp"], {"width": width, "heads": heads}))
    non_emb = 12 * width * width * layers
    total = non_emb + 2 * width * table["vocab"]
    return {"n_head": heads, "n_layer": layers, "n_embd": width, "mlp_hidden_dim": mlp,
            "qkv_dim": r["head_dim"], "head_dim": r["head_dim"],
            "non_emb_params": non_emb, "total_params": total}


def _pick_kappa(sub: dict, kappa) -> list:
    kappa = 0.85 if kappa is None else float(kappa)
    for key in (f"{kappa:.2f}", str(kappa)):
        if key in sub:
            return sub[key]
    nearest = min(sub, key=lambda k: abs(float(k) - kappa))
    return sub[nearest]


def compute_lr(rule_name: str, optimizer_name: str, non_emb_params: float, kappa=None, batch_size=None):
    laws = load_rules()["rules"][rule_name]["lr_laws"]
    base = laws.get(32, {})
    table = laws.get(512, base) if batch_size == 512 else base
    if optimizer_name not in table:
        table = base
    if optimizer_name not in table:
        return None
    entry = table[optimizer_name]
    coeffs = _pick_kappa(entry, kappa) if isinstance(entry, dict) else entry
    if coeffs is None or any(c is None for c in coeffs):
        return compute_lr(rule_name, optimizer_name, non_emb_params, kappa) if table is not base else None
    a, b, d = (float(c) for c in coeffs)  # PyYAML reads '1.67e4' as a string
    return a * (b + non_emb_params) ** d


def apply_scaling_rule(args, verbose: bool = True) -> None:
    """Fill model shape, LR and Chinchilla iteration count (20 tokens/param) into `args`."""
    rule_name = getattr(args, "scaling_rule", "none")
    if rule_name in (None, "none"):
        return
    if args.heads is None:
        raise ValueError("--heads is required when --scaling_rule is set")
    dims = compute_dimensions(rule_name, args.heads)
    rule = load_rules()["rules"][rule_name]
    args.model = rule["model"]
    for k in ("n_head", "n_layer", "n_embd", "mlp_hidden_dim", "qkv_dim"):
        setattr(args, k, dims[k])
    args.weight_tying = bool(rule.get("weight_tying", False))
    lr = compute_lr(rule_name, args.opt, dims["non_emb_params"], kappa=getattr(args, "kappa", None))
    if lr is not None:
        args.lr = lr
    tokens_per_step = args.batch_size * args.acc_steps * args.sequence_length
    args.iterations = int(20 * dims["total_params"] / tokens_per_step)
    if verbose:
        print(f"[Scaling Rule: {rule_name}] heads={args.heads}")
        print(f"  n_head={args.n_head}, n_layer={args.n_layer}, n_embd={args.n_embd}")
        print(f"  mlp_hidden_dim={args.mlp_hidden_dim}, qkv_dim={args.qkv_dim}")
        print(f"  non_emb_params={dims['non_emb_params']:,.0f} ({dims['non_emb_params'] / 1e6:.1f}M)")
        print(f"  total_params={dims['total_params']:,.0f} ({dims['total_params'] / 1e6:.1f}M)")
        print(f"  lr={args.lr:.6e}, iterations={args.iterations}")
