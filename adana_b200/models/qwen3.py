"""Qwen3-style decoder: RMSNorm (or LayerNorm), separate q/k/v/o projections, per-head QK-norm,
RoPE, SwiGLU MLP, optional element-wise sigmoid output gate on the attention output.

Reference parity (src/models/qwen3.py:19-453): MHA, theta = 1e4, gate packed into `q_proj` as
[q_h | gate_h] per head.  Extensions on top: grouped-query attention (`--n_kv_head`) and a
configurable `--rope_theta`.  Parameter names: transformer.h.{i}.{ln_1, ln_2}.weight,
attn.{q_proj, k_proj, v_proj, o_proj}.weight, attn.{q_norm, k_norm}.weight,
mlp.{gate_proj, up_proj, down_proj}.weight, transformer.ln_f.weight, lm_head.weight.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint as _checkpoint

from ..ops.rope import precompute_freqs_cis
from .common import BaseLM, cfg_get, depth_scaled_init_, init_module_weights, make_norm
from .enoki import apply_rotary_emb


class Qwen3MLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        hidden = cfg_get(config, "mlp_hidden_dim", None)
        if hidden is None:
            hidden = int(2 * (4 * config.n_embd) / 3)
            hidden = config.multiple_of * ((hidden + config.multiple_of - 1) // config.multiple_of)
        self.gate_proj = nn.Linear(config.n_embd, hidden, bias=config.bias)
        self.up_proj = nn.Linear(config.n_embd, hidden, bias=config.bias)
        self.down_proj = nn.Linear(hidden, config.n_embd, bias=config.bias)
        self.dropout = nn.Dropout(config.dropout)

    def forward(self, x):
        return self.dropout(self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))), {}


class Qwen3Attention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.qkv_dim = cfg_get(config, "qkv_dim", config.n_embd // config.n_head)
        self.n_head = config.n_head
        self.n_kv_head = cfg_get(config, "n_kv_head", config.n_head)
        assert self.n_head % self.n_kv_head == 0
        self.gate = bool(cfg_get(config, "elementwise_attn_output_gate", False))
        q_out = self.n_head * self.qkv_dim
        kv_out = self.n_kv_head * self.qkv_dim
        self.q_proj = nn.Linear(config.n_embd, (2 if self.gate else 1) * q_out, bias=config.bias)
        self.k_proj = nn.Linear(config.n_embd, kv_out, bias=config.bias)
        self.v_proj = nn.Linear(config.n_embd, kv_out, bias=config.bias)
        self.o_proj = nn.Linear(q_out, config.n_embd, bias=config.bias)
        self.resid_dropout = nn.Dropout(config.dropout)
        self.dropout = config.dropout
        self.use_qknorm = not cfg_get(config, "no_qknorm", False)
        if self.use_qknorm:
            kind = cfg_get(config, "normalization_layer_type", "rmsnorm")
            self.q_norm = make_norm(kind, self.qkv_dim, config.bias, cfg_get(config, "rmsnorm_eps", 1e-5))
            self.k_norm = make_norm(kind, self.qkv_dim, config.bias, cfg_get(config, "rmsnorm_eps", 1e-5))

    def forward(self, x, freqs_cis):
        B, T, _ = x.shape
        q = self.q_proj(x)
        k = self.k_proj(x).view(B, T, -1, self.qkv_dim)
        v = self.v_proj(x).view(B, T, -1, self.qkv_dim)
        gate = None
        if self.gate:
            q, gate = q.view(B, T, -1, 2 * self.qkv_dim).split([self.qkv_dim, self.qkv_dim], dim=-1)
        else:
            q = q.view(B, T, -1, self.qkv_dim)
        if self.use_qknorm:
            q, k = self.q_norm(q), self.k_norm(k)
        q, k = apply_rotary_emb(q, k, freqs_cis)
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        if q.dtype != v.dtype:
            q, k = q.to(v.dtype), k.to(v.dtype)
        y = F.scaled_dot_product_attention(q, k, v, attn_mask=None, is_causal=True,
                                           dropout_p=self.dropout if self.training else 0.0,
                                           enable_gqa=self.n_kv_head != self.n_head)
        y = y.transpose(1, 2).contiguous()
        if gate is not None:
            y = y * torch.sigmoid(gate)
        return self.resid_dropout(self.o_proj(y.view(B, T, -1)))


class Qwen3Block(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        kind = cfg_get(config, "normalization_layer_type", "rmsnorm")
        eps = cfg_get(config, "rmsnorm_eps", 1e-5)
        self.ln_1 = make_norm(kind, config.n_embd, config.bias, eps)
        self.attn = Qwen3Attention(config)
        self.ln_2 = make_norm(kind, config.n_embd, config.bias, eps)
        if cfg_get(config, "moe", False):
            from .moe import MoE

            self.mlp = MoE(config, Qwen3MLP)
        else:
            self.mlp = Qwen3MLP(config)
        self.scale = cfg_get(config, "residual_stream_scalar", 1.0)

    def forward(self, x, freqs_cis):
        x = x + self.scale * self.attn(self.ln_1(x), freqs_cis)
        y, extra = self.mlp(self.ln_2(x))
        return x + self.scale * y, extra


class Qwen3(BaseLM):
    arch = "qwen3"
    block_cls = Qwen3Block
    residual_out_suffixes = ("o_proj.weight", "down_proj.weight")

    def __init__(self, config):
        super().__init__(config)
        self.head_dim = cfg_get(config, "qkv_dim", config.n_embd // config.n_head)
        self.freqs_cis = precompute_freqs_cis(self.head_dim, config.sequence_length,
                                              cfg_get(config, "rope_theta", 10000.0))
        kind = cfg_get(config, "normalization_layer_type", "rmsnorm")
        self.transformer = nn.ModuleDict(dict(
            wte=nn.Embedding(config.vocab_size, config.n_embd),
            drop=nn.Dropout(config.dropout),
            h=nn.ModuleList([self.block_cls(config) for _ in range(config.n_layer)]),
            ln_f=make_norm(kind, config.n_embd, config.bias, cfg_get(config, "rmsnorm_eps", 1e-5)),
        ))
        self.lm_head = nn.Linear(config.n_embd, config.vocab_size, bias=False)
        if config.weight_tying:
            self.transformer.wte.weight = self.lm_head.weight
        scheme, std = cfg_get(config, "init_scheme", "KarpathyGPT2"), cfg_get(config, "init_std", 0.02)
        if cfg_get(config, "init_compat", "none") == "reference" and self.arch == "qwen3":
            from .init_compat import reference_compatible_init_

            reference_compatible_init_(self, config, "qwen3", tuple(self.residual_out_suffixes))
        else:
            self.apply(lambda m: init_module_weights(m, scheme, std))
            depth_scaled_init_(self.named_parameters(), self.residual_out_suffixes, scheme, std, config.n_layer)

    @staticmethod
    def get_tp_plan():
        return {"attn.q_proj": "colwise", "attn.k_proj": "colwise", "attn.v_proj": "colwise",
                "attn.o_proj": "rowwise", "mlp.gate_proj": "colwise", "mlp.up_proj": "colwise",
                "mlp.down_proj": "rowwise"}

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
