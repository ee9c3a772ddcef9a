"""Model-size arithmetic of the scaling studies: parameter counts of every scaling rule the sweeps used, the
training-compute formulas that the loss laws are fitted against, and the Chinchilla iteration budget.

The reference repeats this arithmetic inside each figure script (visualization/compare_scaling_rules_ep.py:238-392,
bighead_lr_scaling.py:222-341, gamma3_factor_scaling.py:119-164, hoyer_final_loss.py:100-143); here it is one table.
A rule maps the sweep's size knob (depth for BigHead, heads for the others) to (layers, heads, width, non-embedding
parameters); total parameters add the untied embedding and LM head (2 * width * 50304).

Compute formulas, with D = 20 * total parameters tokens:
  default  6 * non_emb * D
  6N1      72 * layers * width^2 * D                          (Kaplan: matrices only)
  6N2      (72 * layers * width^2 + 6 * vocab * width) * D    (Chinchilla: with the LM head)
  M        (72 * layers * width^2 + 12 * layers * width * S) * D   (DeepSeek: with attention over S positions)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict

VOCAB = 50304
PFH = 3600e15            # FLOPs in one PetaFLOP-hour
PF_DAY = 1e15 * 86400    # FLOPs in one PetaFLOP-day
TOKENS_PER_ITERATION = 65536   # 32 sequences of 2048 tokens: the batch of the sweeps


@dataclass(frozen=True)
class ModelSize:
    rule: str
    size: int
    n_layer: int
    n_head: int
    n_embd: int
    non_emb: int
    total_params: int

    @property
    def chinchilla_tokens(self) -> float:
        return 20.0 * self.total_params

    def flops_per_token(self, formula: str = "default", seq_length: int = 2048) -> float:
        mats = 72.0 * self.n_layer * self.n_embd * self.n_embd
        if formula == "default":
            return 6.0 * self.non_emb
        if formula == "6N1":
            return mats
        if formula == "6N2":
            return mats + 6.0 * VOCAB * self.n_embd
        if formula == "M":
            return mats + 12.0 * self.n_layer * self.n_embd * seq_length
        raise ValueError(f"unknown compute formula {formula!r} (default, 6N1, 6N2, M)")

    def compute_pfh(self, formula: str = "default", seq_length: int = 2048) -> float:
        """Compute of the Chinchilla-budget run in PetaFLOP-hours."""
        return self.flops_per_token(formula, seq_length) * self.chinchilla_tokens / PFH

    def chinchilla_iterations(self, tokens_per_iteration: int = TOKENS_PER_ITERATION) -> int:
        return int(20 * self.total_params / tokens_per_iteration)

    def flops_per_iteration(self, batch_size: int = 1, seq_len: int = 512) -> float:
        """6 * non_emb per token: what the loss-curve figures put on their compute axis."""
        return 6.0 * float(self.non_emb) * float(seq_len) * float(batch_size)


def _gpt_block(n_layer, n_head, head_dim, n_embd, mlp_hidden):
    # fused qkv + projection + two MLP matrices + the eight per-block vectors, plus the final norm's two
    return n_layer * (3 * head_dim * n_embd * n_head + n_embd * n_embd + 2 * n_embd * mlp_hidden + 8 * n_embd) + 2 * n_embd


def _bighead(d):
    return d, d, 16 * d * d, _gpt_block(d, d, 16 * d, 16 * d * d, 32 * d * d)


def _egghead(h):
    L = int(h * (h - 1) / 2)
    return L, h, 16 * h * h, _gpt_block(L, h, 16 * h, 16 * h * h, 32 * h * h)


def _enoki(h):
    L, d = int(3 * h // 4), 64 * h
    return L, h, d, 12 * d * d * L


def _eryngii(h):
    hd = int(round(32 * h / 3 / 8) * 8)
    L, d = int(h * h // 8), h * hd
    return L, h, d, 12 * d * d * L


def _qwen3(h):
    hd, L, d = 128, 2 * h, 128 * h
    per_layer = 5 * d * (h * hd) + 2 * hd + 9 * d * d + 2 * d      # gated q (2x), k, v, o; QK-norms; SwiGLU 3d; two norms
    return L, h, d, L * per_layer + d


RULES: Dict[str, Callable] = {
    "BigHead": _bighead, "EggHead": _egghead,
    "Enoki": _enoki, "Enoki_Scaled": _enoki, "Enoki_512": _enoki,
    "Eryngii": _eryngii, "Eryngii_Scaled": _eryngii,
    "Qwen3_Scaled": _qwen3, "Qwen3_Hoyer": _qwen3,
}


def model_size(size: int, rule: str = "Enoki_Scaled") -> ModelSize:
    try:
        fn = RULES[rule]
    except KeyError:
        raise ValueError(f"unknown scaling rule {rule!r}; known: {sorted(RULES)}") from None
    L, H, d, non_emb = fn(int(size))
    return ModelSize(rule, int(size), int(L), int(H), int(d), int(non_emb), int(non_emb + 2 * d * VOCAB))


def size_key(rule: str) -> str:
    """Name of the config entry that holds the sweep's size knob."""
    return "n_layer" if rule == "BigHead" else "n_head"


def petaflop_days(flops: float) -> float:
    return flops / PF_DAY
