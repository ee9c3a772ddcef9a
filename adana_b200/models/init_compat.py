"""Seed-compatible initialisation: make a model's initial weights bit-identical to what the reference
builds from the same `--seed`, so loss curves can be compared step by step rather than statistically.

The reference draws from the global CPU generator while it constructs a model, and its decoders are built
in two rounds (src/models/base.py:166-212 builds and initialises a GPT-2-style network, then
src/models/enoki.py:203-237 / src/models/qwen3.py:271-310 replace its blocks and initialise again).  Only
the second round's values survive, but they depend on how many numbers the first round consumed.  This module
does not replay that code: it *burns* the same number of uniform / normal draws from a private generator
(`prelude`, a list of (distribution, count) derived from the configuration) and then initialises the real
parameters in module order from that generator.  Counts, not shapes, matter: a CPU `uniform_` / `normal_`
of n elements advances the generator identically for any shape.

Enabled with `--init_compat reference`; covered: enoki / diloco and qwen3 without MoE and with as many KV
heads as query heads (the reference has no grouped-query attention).  The test compares against golden
checksums and losses produced by the reference.
"""
from __future__ import annotations

import math
from typing import Iterator, List, Tuple

import torch
import torch.nn as nn


def _lin(n_in: int, n_out: int, bias: bool) -> List[Tuple[str, int]]:
    """nn.Linear's constructor: kaiming-uniform weight, uniform bias."""
    return [("uniform", n_in * n_out)] + ([("uniform", n_out)] if bias else [])


def prelude(config, arch: str) -> Iterator[Tuple[str, int]]:
    """(distribution, count) of every draw the reference makes before its final initialisation pass."""
    V, d, S, L = config.vocab_size, config.n_embd, config.sequence_length, config.n_layer
    bias = bool(getattr(config, "bias", False))
    scheme = getattr(config, "init_scheme", "KarpathyGPT2")
    if getattr(config, "moe", False):
        raise NotImplementedError("--init_compat reference does not cover MoE models")
    # round one: GPT-2-style network (token + position embeddings, fused-QKV attention, 4x GELU MLP, head)
    yield ("normal", V * d)
    yield ("normal", S * d)
    for _ in range(L):
        for n_in, n_out in ((d, 3 * d), (d, d), (d, 4 * d), (4 * d, d)):
            yield from _lin(n_in, n_out, bias)
    yield from _lin(d, V, False)
    yield ("normal", V * d)
    yield ("normal", S * d)
    for _ in range(L):
        for n in (3 * d * d, d * d, 4 * d * d, 4 * d * d):
            yield ("normal", n)
    yield ("normal", V * d)
    if scheme == "KarpathyGPT2":
        for _ in range(L):
            yield ("normal", d * d)
            yield ("normal", 4 * d * d)
    # round two, construction of the architecture's own blocks
    hd = getattr(config, "qkv_dim", None) or d // config.n_head
    Q = hd * config.n_head
    hidden = getattr(config, "mlp_hidden_dim", None)
    if arch in ("enoki", "diloco"):
        if hidden is None:
            hidden = int(2 * (4 * d) / 3)
            hidden = config.multiple_of * ((hidden + config.multiple_of - 1) // config.multiple_of)
        for _ in range(L):
            # its block class extends the GPT-2 block: that block's four projections are built first
            for n_in, n_out in ((d, 3 * d), (d, d), (d, 4 * d), (4 * d, d), (d, 3 * Q), (Q, d), (d, hidden), (hidden, d)):
                yield from _lin(n_in, n_out, bias)
    elif arch == "qwen3":
        if getattr(config, "n_kv_head", None) not in (None, config.n_head):
            raise NotImplementedError("--init_compat reference needs n_kv_head == n_head")
        if hidden is None:
            hidden = int(2 * (4 * d) / 3)
            hidden = config.multiple_of * ((hidden + config.multiple_of - 1) // config.multiple_of)
        gate = 2 if getattr(config, "elementwise_attn_output_gate", False) else 1
        for _ in range(L):
            for n_in, n_out in ((d, gate * Q), (d, Q), (d, Q), (Q, d), (d, hidden), (d, hidden), (hidden, d)):
                yield from _lin(n_in, n_out, bias)
    else:
        raise NotImplementedError(f"--init_compat reference does not cover --model {arch}")


def _burn(gen: torch.Generator, kind: str, count: int, scratch: torch.Tensor) -> None:
    t = scratch[:count]
    if kind == "uniform":
        t.uniform_(-1.0, 1.0, generator=gen)
    else:
        t.normal_(generator=gen)


def _post_order(module: nn.Module):
    for child in module.children():
        yield from _post_order(child)
    yield module


@torch.no_grad()
def reference_compatible_init_(model: nn.Module, config, arch: str, depth_scaled_suffixes: Tuple[str, ...]) -> None:
    seed = int(getattr(config, "seed", 0))
    gen = torch.Generator(device="cpu").manual_seed(seed)
    draws = list(prelude(config, arch))
    scratch = torch.empty(max(n for _, n in draws), dtype=torch.float32)
    for kind, n in draws:
        _burn(gen, kind, n, scratch)
    del scratch
    scheme = getattr(config, "init_scheme", "KarpathyGPT2")
    std0 = getattr(config, "init_std", 0.02)

    def draw_into(p: torch.Tensor, std: float):
        tmp = torch.empty(p.shape, dtype=torch.float32).normal_(0.0, std, generator=gen)
        p.copy_(tmp)

    done = set()
    for mod in _post_order(model):
        if isinstance(mod, nn.Linear):
            std = 1.0 / math.sqrt(mod.weight.size(1)) if scheme in ("Standard", "ScaledGPT") else std0
            draw_into(mod.weight, std)          # tied weights are drawn once per module that holds them
            if mod.bias is not None:
                mod.bias.zero_()
        elif isinstance(mod, nn.Embedding):
            std = {"Standard": 1.0, "ScaledGPT": 1.0 / math.sqrt(mod.weight.size(1))}.get(scheme, std0)
            draw_into(mod.weight, std)
        done.add(id(mod))
    for name, p in model.named_parameters():
        if name.endswith(depth_scaled_suffixes):
            if scheme == "KarpathyGPT2":
                draw_into(p, std0 / math.sqrt(2 * config.n_layer))
            elif scheme == "ScaledGPT":
                draw_into(p, 1.0 / math.sqrt(2 * p.size(1) * config.n_layer))
