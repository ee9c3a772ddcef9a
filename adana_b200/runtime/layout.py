"""Flat-buffer layout of a model for the kernel engine.

A model is cut into *units* (one per transformer block plus a root unit holding the token
embedding, the final norm and the LM head) — the same grouping the reference hands to FSDP2
(src/distributed/fsdp.py:105-116).  Inside a unit the parameters are laid out back to back in
one flat buffer, in an order chosen for the kernels rather than for the module tree:

  * matrices that are consumed by ONE fused GEMM are adjacent (Qwen3 q|k|v projections form one
    [Nq+2Nkv, d] operand, gate|up one [2*mlp, d] operand), so fusing costs no copy;
  * weight-decayed parameters come first, then the non-decayed ones, so that the optimizer
    kernel runs over two contiguous ranges per unit;
  * every slot starts on a 64-element boundary (TMA needs 16-byte aligned bases) and the unit is
    padded to a multiple of `64 * world_size` so that it splits evenly into rank shards.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

ALIGN = 64


@dataclass
class Slot:
    name: str                 # fully qualified parameter name in the module tree
    shape: Tuple[int, ...]
    offset: int               # element offset inside the unit's flat buffer
    decay: bool

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


@dataclass
class UnitLayout:
    name: str
    slots: List[Slot] = field(default_factory=list)
    numel: int = 0            # used elements (before padding)
    padded: int = 0           # multiple of ALIGN * world
    decay_end: int = 0        # [0, decay_end) decays, [decay_end, numel) does not

    def slot(self, suffix: str) -> Slot:
        for s in self.slots:
            if s.name.endswith(suffix):
                return s
        raise KeyError(f"{self.name}: no parameter ending in {suffix}")

    def has(self, suffix: str) -> bool:
        return any(s.name.endswith(suffix) for s in self.slots)


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def _build_unit(name: str, named: List[Tuple[str, torch.Tensor]], order: List[str], decay_names: set,
                world: int) -> UnitLayout:
    by_suffix = dict(named)
    decay_list = [n for n in order if n in by_suffix and n in decay_names]
    nodecay_list = [n for n in order if n in by_suffix and n not in decay_names]
    missing = set(by_suffix) - set(order)
    if missing:
        raise ValueError(f"unit {name}: parameters without a layout position: {sorted(missing)}")
    u = UnitLayout(name=name)
    off = 0
    for n in decay_list:
        u.slots.append(Slot(n, tuple(by_suffix[n].shape), off, True))
        off = _round_up(off + by_suffix[n].numel(), ALIGN)
    u.decay_end = off
    for n in nodecay_list:
        u.slots.append(Slot(n, tuple(by_suffix[n].shape), off, False))
        off = _round_up(off + by_suffix[n].numel(), ALIGN)
    u.numel = off
    u.padded = _round_up(max(off, 1), ALIGN * world)
    return u


ENOKI_BLOCK_ORDER = ["attn.c_attn.weight", "attn.c_proj.weight", "mlp.c_fc.weight", "mlp.c_proj.weight",
                     "ln_1.weight", "ln_2.weight", "attn.q_layernorm.weight", "attn.k_layernorm.weight"]
QWEN3_BLOCK_ORDER = ["attn.q_proj.weight", "attn.k_proj.weight", "attn.v_proj.weight", "attn.o_proj.weight",
                     "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight",
                     "ln_1.weight", "ln_2.weight", "attn.q_norm.weight", "attn.k_norm.weight"]
LLAMA_BLOCK_ORDER = ["attn.c_attn.weight", "attn.c_proj.weight", "mlp.w1.weight", "mlp.w2.weight", "mlp.c_proj.weight",
                     "ln_1.weight", "ln_2.weight"]
BLOCK_ORDERS = {"enoki": ENOKI_BLOCK_ORDER, "qwen3": QWEN3_BLOCK_ORDER, "llama": LLAMA_BLOCK_ORDER}
ROOT_ORDER = ["lm_head.weight", "transformer.wte.weight", "transformer.ln_f.weight"]


def build_layouts(model, world: int) -> List[UnitLayout]:
    """Units in execution order: blocks 0..L-1, then the root unit (last)."""
    arch = getattr(model, "arch", None)
    if arch not in BLOCK_ORDERS:
        raise ValueError(f"kernel engine supports enoki, qwen3 and llama models, got {arch!r}")
    specs = model.get_parameter_group_specs()
    decay_names = set(specs[0]["params"])
    order = BLOCK_ORDERS[arch]
    units: List[UnitLayout] = []
    for i, blk in enumerate(model.transformer.h):
        prefix = f"transformer.h.{i}."
        named = [(prefix + n, p) for n, p in blk.named_parameters()]
        units.append(_build_unit(f"block{i}", named, [prefix + n for n in order], decay_names, world))
    root_named = [(n, p) for n, p in model.named_parameters() if not n.startswith("transformer.h.")]
    units.append(_build_unit("root", root_named, ROOT_ORDER, decay_names, world))
    return units


def engine_supported(model, cfg) -> Optional[str]:
    """None when the kernel engine can run this model, else the reason it cannot."""
    if getattr(model, "arch", None) not in BLOCK_ORDERS:
        return f"architecture {type(model).__name__} has no kernel path"
    if getattr(cfg, "bias", False):
        return "bias terms are not supported by the kernel path"
    if getattr(cfg, "dropout", 0.0) != 0.0:
        return "dropout is not supported by the kernel path"
    if getattr(cfg, "moe", False):
        return "MoE blocks run on the PyTorch path"
    if getattr(cfg, "weight_tying", False) and model.arch == "qwen3":
        return "tied embeddings run on the PyTorch path"
    hd = getattr(model, "head_dim", 0)
    if hd % 2:
        return "odd head dimension"
    return None
