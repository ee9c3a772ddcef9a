"""Enoki: GPT-style decoder with RoPE, per-head QK-LayerNorm, GELU MLP, weight-only LayerNorm,
untied embeddings and a z-loss on the logits (`--model enoki`; `diloco` is the same network).

Parameter names and shapes follow the reference (src/models/enoki.py:64-237) so checkpoints
interchange:  transformer.wte.weight [V,d]; transformer.h.{i}.{ln_1.weight, attn.c_attn.weight
[3*H*hd, d] (rows q|k|v, head-major), attn.c_proj.weight [d, H*hd], attn.q_layernorm.weight
[hd], attn.k_layernorm.weight [hd], ln_2.weight, mlp.c_fc.weight [mlp, d], mlp.c_proj.weight
[d, mlp]}; transformer.ln_f.weight; lm_head.weight [V,d].

`forward` is the PyTorch path (autograd; runs anywhere, fp32 or autocast).  When a kernel
engine is attached (`adana_b200.runtime.engine`), training forwards go through the
hand-written sm_100a kernels instead; both paths use the same parameters.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint as _checkpoint

from ..ops.rope import precompute_freqs_cis
from .common import BaseLM, LayerNorm, cfg_get, depth_scaled_init_, init_module_weights


def apply_rotary_emb(q, k, freqs_cis):
    """Interleaved-pair rotation in fp32.  q,k [B,T,H,hd]; freqs_cis [T, hd/2, 2] -> fp32 q,k."""
    def rot(x):
        xr = x.float().reshape(*x.shape[:-1], -1, 2)
        f = freqs_cis.view(1, xr.shape[1], 1, xr.shape[3], 2)
        o0 = xr[..., 0] * f[..., 0] - xr[..., 1] * f[..., 1]
        o1 = xr[..., 0] * f[..., 1] + xr[..., 1] * f[..., 0]
        return torch.stack((o0, o1), dim=-1).flatten(3)
    return rot(q), rot(k)


class EnokiAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.qkv_dim = cfg_get(config, "qkv_dim", config.n_embd // config.n_head)
        self.total_qkv_dim = self.qkv_dim * config.n_head
        self.c_attn = nn.Linear(config.n_embd, 3 * self.total_qkv_dim, bias=config.bias)
        self.c_proj = nn.Linear(self.total_qkv_dim, config.n_embd, bias=config.bias)
        self.resid_dropout = nn.Dropout(config.dropout)
        self.n_head = config.n_head
        self.dropout = config.dropout
        self.use_qknorm = not cfg_get(config, "no_qknorm", False)
        if self.use_qknorm:
            self.q_layernorm = LayerNorm(self.qkv_dim, bias=config.bias)
            self.k_layernorm = LayerNorm(self.qkv_dim, bias=config.bias)

    def forward(self, x, freqs_cis):
        B, T, _ = x.shape
        q, k, v = self.c_attn(x).chunk(3, dim=-1)
        q = q.view(B, T, -1, self.qkv_dim)
        k = k.view(B, T, -1, self.qkv_dim)
        v = v.view(B, T, -1, self.qkv_dim)
        if self.use_qknorm:
            q, k = self.q_layernorm(q), self.k_layernorm(k)
        q, k = apply_rotary_emb(q, k, freqs_cis)
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        if q.dtype != v.dtype:  # rotated q,k are fp32; match the value dtype under autocast
            q, k = q.to(v.dtype), k.to(v.dtype)
        y = F.scaled_dot_product_attention(q, k, v, attn_mask=None,
                                           dropout_p=self.dropout if self.training else 0.0, is_causal=True)
        y = y.transpose(1, 2).contiguous().view(B, T, -1)
        return self.resid_dropout(self.c_proj(y))


class EnokiMLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        hidden = cfg_get(config, "mlp_hidden_dim", None)
        if hidden is None:
            hidden = int(2 * (4 * config.n_embd) / 3)
            hidden = config.multiple_of * ((hidden + config.multiple_of - 1) // config.multiple_of)
        self.c_fc = nn.Linear(config.n_embd, hidden, bias=config.bias)
        self.c_proj = nn.Linear(hidden, config.n_embd, bias=config.bias)
        self.dropout = nn.Dropout(config.dropout)
        self.activation = nn.GELU()

    def forward(self, x):
        return self.dropout(self.c_proj(self.activation(self.c_fc(x)))), {}


class EnokiBlock(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.ln_1 = LayerNorm(config.n_embd, bias=config.bias)
        self.attn = EnokiAttention(config)
        self.ln_2 = LayerNorm(config.n_embd, bias=config.bias)
        if cfg_get(config, "moe", False):
            from .moe import MoE

            self.mlp = MoE(config, EnokiMLP)
        else:
            self.mlp = EnokiMLP(config)
        self.scale = cfg_get(config, "residual_stream_scalar", 1.0)

    def forward(self, x, freqs_cis):
        x = x + self.scale * self.attn(self.ln_1(x), freqs_cis)
        y, extra = self.mlp(self.ln_2(x))
        return x + self.scale * y, extra


class Enoki(BaseLM):
    arch = "enoki"

    def __init__(self, config):
        config.weight_tying = False
        super().__init__(config)
        self.head_dim = cfg_get(config, "qkv_dim", config.n_embd // config.n_head)
        self.freqs_cis = precompute_freqs_cis(self.head_dim, config.sequence_length,
                                              cfg_get(config, "rope_theta", 10000.0))
        self.transformer = nn.ModuleDict(dict(
            wte=nn.Embedding(config.vocab_size, config.n_embd),
            drop=nn.Dropout(config.dropout),
            h=nn.ModuleList([EnokiBlock(config) for _ in range(config.n_layer)]),
            ln_f=LayerNorm(config.n_embd, bias=config.bias),
        ))
        self.lm_head = nn.Linear(config.n_embd, config.vocab_size, bias=False)
        scheme, std = cfg_get(config, "init_scheme", "KarpathyGPT2"), cfg_get(config, "init_std", 0.02)
        if cfg_get(config, "init_compat", "none") == "reference":
            from .init_compat import reference_compatible_init_

            reference_compatible_init_(self, config, "enoki", ("c_proj.weight",))
        else:
            self.apply(lambda m: init_module_weights(m, scheme, std))
            depth_scaled_init_(self.named_parameters(), ("c_proj.weight",), scheme, std, config.n_layer)

    @staticmethod
    def get_tp_plan():
        """Block-relative module path -> 'colwise' | 'rowwise' (see parallel/tensor_parallel.py)."""
        return {"attn.c_attn": "colwise", "attn.c_proj": "rowwise",
                "mlp.c_fc": "colwise", "mlp.c_proj": "rowwise"}

    def get_num_params(self, non_embedding=True, exclude_embeddings=False):
        n = sum(p.numel() for p in self.parameters())
        if exclude_embeddings:
            n -= self.transformer.wte.weight.numel() + self.lm_head.weight.numel()
        return n

    def forward(self, idx, targets=None, get_logits=False, moe=False, compute_accuracy=False):
        if self._engine is not None and self._engine.handles(self, idx, targets, get_logits):
            return self._engine.forward(idx, targets, compute_accuracy=compute_accuracy)
        cfg = self.config
        b, t = idx.shape
        assert t <= cfg.sequence_length, \
            f"Cannot forward sequence of length {t}, block size is only {cfg.sequence_length}"
        tok_emb = self.transformer.wte(idx)
        x = self.transformer.drop(tok_emb)
        freqs = self.freqs_cis.to(x.device)[:t]
        router_logits, experts = [], []
        ckpt = cfg_get(cfg, "activation_checkpointing", False)
        every = cfg_get(cfg, "checkpoint_every_n", 1)
        for i, block in enumerate(self.transformer.h):
            if ckpt and self.training and i % every == 0:
                x, extra = _checkpoint(block, x, freqs, use_reentrant=False)
            else:
                x, extra = block(x, freqs)
            if extra:
                router_logits.append(extra["router_logits"])
                experts.append(extra["selected_experts"])
        x = self.transformer.ln_f(x)
        aux, acc, logits, loss = {}, None, None, None
        if targets is not None:
            loss, logits, aux, acc = self._loss_head(x, tok_emb, targets, get_logits, compute_accuracy)
            if moe and cfg_get(cfg, "moe_routing", None) == "standard_gating":
                from .moe import router_losses

                for lg, ex in zip(router_logits, experts):
                    for k, v in router_losses(cfg, lg, ex, eval_mode=not self.training).items():
                        aux[k] = aux.get(k, 0.0) + v
                        if self.training:
                            loss = loss + v * getattr(cfg, k + "_factor") / cfg.n_layer
        else:
            logits = self.lm_head(x[:, [-1], :])
        return {"logits": logits if get_logits else None, "loss": loss, "aux_losses": aux,
                "router_logits": torch.stack(router_logits, 0) if router_logits else None,
                "accuracy": acc}


DiLoCo = Enoki  # legacy alias (`--model diloco`): same network with hard-coded head counts upstream
