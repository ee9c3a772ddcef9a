"""Qwen3Next (`--model qwen3next`): Qwen3 blocks whose MLP is, layer by layer, either dense or a
routed MoE plus a sigmoid-gated shared expert.  A layer is sparse when `--moe` is set, the layer is
not listed in `--mlp_only_layers`, and `layer % decoder_sparse_step == 0`
(reference: src/models/qwen3next.py:20-261).  With several ranks and `--expert_parallel` the routed
experts are sharded over the ranks (`adana_b200/parallel/expert_parallel.py`).
"""
from __future__ import annotations

import copy

import torch
import torch.distributed as dist
import torch.nn as nn

from .common import cfg_get, make_norm
from .moe import MoE
from .qwen3 import Qwen3, Qwen3Attention, Qwen3MLP


def _dense_only_layers(config):
    v = cfg_get(config, "mlp_only_layers", None)
    if v is None:
        return []
    if isinstance(v, str):
        return [int(x) for x in v.split(",") if x.strip()]
    return list(v)


class Qwen3NextMoE(nn.Module):
    def __init__(self, config, mlp_class):
        super().__init__()
        self.config = config
        gated = bool(cfg_get(config, "use_gated_shared_expert", False))
        moe_cfg = config
        if gated:
            moe_cfg = copy.copy(config)
            moe_cfg.moe_num_shared_experts = 0
        ep = cfg_get(config, "expert_parallel", True) and dist.is_available() and dist.is_initialized() \
            and dist.get_world_size() > 1
        if ep:
            from ..parallel.expert_parallel import ExpertParallelMoE

            self.routed_moe = ExpertParallelMoE(moe_cfg, mlp_class)
        else:
            self.routed_moe = MoE(moe_cfg, mlp_class)
        self.shared_expert = self.shared_expert_gate = None
        if gated:
            shared_cfg = copy.copy(config)
            if cfg_get(config, "shared_expert_intermediate_size", None) is not None:
                shared_cfg.mlp_hidden_dim = config.shared_expert_intermediate_size
            self.shared_expert = mlp_class(shared_cfg)
            self.shared_expert_gate = nn.Linear(config.n_embd, 1, bias=False)

    def forward(self, x):
        out, info = self.routed_moe(x)
        if self.shared_expert is not None:
            flat = x.view(-1, x.shape[-1])
            shared, _ = self.shared_expert(flat)
            out = out + (torch.sigmoid(self.shared_expert_gate(flat)) * shared).view_as(x)
        return out, info


class Qwen3NextBlock(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.config, self.layer_idx = config, layer_idx
        kind, eps = cfg_get(config, "normalization_layer_type", "rmsnorm"), cfg_get(config, "rmsnorm_eps", 1e-5)
        self.ln_1 = make_norm(kind, config.n_embd, config.bias, eps)
        self.ln_2 = make_norm(kind, config.n_embd, config.bias, eps)
        self.attn = Qwen3Attention(config)
        self.is_moe_layer = self.uses_moe(config, layer_idx)
        self.mlp = Qwen3NextMoE(config, Qwen3MLP) if self.is_moe_layer else Qwen3MLP(config)
        self.scale = cfg_get(config, "residual_stream_scalar", 1.0)

    @staticmethod
    def uses_moe(config, layer_idx: int) -> bool:
        if layer_idx in _dense_only_layers(config) or not cfg_get(config, "moe", False):
            return False
        return layer_idx % cfg_get(config, "decoder_sparse_step", 1) == 0

    def forward(self, x, freqs_cis):
        x = x + self.scale * self.attn(self.ln_1(x), freqs_cis)
        y, extra = self.mlp(self.ln_2(x))
        return x + self.scale * y, extra


class Qwen3Next(Qwen3):
    arch = "qwen3next"

    def __init__(self, config):
        counter = iter(range(10 ** 9))
        type(self).block_cls = staticmethod(lambda cfg: Qwen3NextBlock(cfg, next(counter)))
        super().__init__(config)
        type(self).block_cls = Qwen3NextBlock

    def print_sparsity_pattern(self):
        marks = ["MoE  " if b.is_moe_layer else "dense" for b in self.transformer.h]
        print("Qwen3Next layer pattern: " + " ".join(f"{i}:{m}" for i, m in enumerate(marks)))
        return marks
