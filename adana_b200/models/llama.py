"""Llama-style decoder (`--model llama`): RMSNorm (eps `--rmsnorm_eps`), RoPE, fused QKV, SwiGLU MLP
whose width is 8/3·d rounded up to `--multiple_of`, always-tied embeddings.  Names as in the
reference (src/models/llama.py:66-215): attn.{c_attn,c_proj}, mlp.{w1,w2,c_proj}.  Dense models run on the kernel
engine (RMSNorm, fused q|k|v, RoPE without a per-head norm, SwiGLU over the adjacent w1 | w2, one table as embedding and
LM head); MoE variants on the PyTorch path.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint as _checkpoint

from ..ops.rope import precompute_freqs_cis
from .common import BaseLM, RMSNorm, cfg_get, init_module_weights
from .enoki import apply_rotary_emb


class LlamaMLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        hidden = int(2 * (4 * config.n_embd) / 3)
        hidden = config.multiple_of * ((hidden + config.multiple_of - 1) // config.multiple_of)
        self.w1 = nn.Linear(config.n_embd, hidden, bias=False)
        self.w2 = nn.Linear(config.n_embd, hidden, bias=False)
        self.c_proj = nn.Linear(hidden, config.n_embd, bias=False)

    def forward(self, x):
        return self.c_proj(F.silu(self.w1(x)) * self.w2(x)), {}


class LlamaAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        assert config.n_embd % config.n_head == 0
        self.c_attn = nn.Linear(config.n_embd, 3 * config.n_embd, bias=config.bias)
        self.c_proj = nn.Linear(config.n_embd, config.n_embd, bias=config.bias)
        self.resid_dropout = nn.Dropout(config.dropout)
        self.n_head, self.dropout = config.n_head, config.dropout

    def forward(self, x, freqs_cis):
        B, T, C = x.shape
        hd = C // self.n_head
        q, k, v = self.c_attn(x).chunk(3, dim=-1)
        q, k = apply_rotary_emb(q.view(B, T, -1, hd), k.view(B, T, -1, hd), freqs_cis)
        v = v.view(B, T, -1, hd).transpose(1, 2)
        q, k = q.transpose(1, 2).to(v.dtype), k.transpose(1, 2).to(v.dtype)
        y = F.scaled_dot_product_attention(q, k, v, attn_mask=None, is_causal=True,
                                           dropout_p=self.dropout if self.training else 0.0)
        return self.resid_dropout(self.c_proj(y.transpose(1, 2).contiguous().view(B, T, -1)))


class LlamaBlock(nn.Module):
    def __init__(self, config):
        super().__init__()
        eps = cfg_get(config, "rmsnorm_eps", 1e-5)
        self.ln_1 = RMSNorm(config.n_embd, eps=eps)
        self.attn = LlamaAttention(config)
        self.ln_2 = RMSNorm(config.n_embd, eps=eps)
        if cfg_get(config, "moe", False):
            from .moe import MoE

            self.mlp = MoE(config, LlamaMLP)
        else:
            self.mlp = LlamaMLP(config)

    def forward(self, x, freqs_cis):
        x = x + self.attn(self.ln_1(x), freqs_cis)
        y, extra = self.mlp(self.ln_2(x))
        return x + y, extra


class Llama(BaseLM):
    arch = "llama"

    def __init__(self, config):
        config.weight_tying = True
        super().__init__(config)
        self.head_dim = config.n_embd // config.n_head
        self.freqs_cis = precompute_freqs_cis(self.head_dim, config.sequence_length,
                                              cfg_get(config, "rope_theta", 10000.0))
        self.transformer = nn.ModuleDict(dict(
            wte=nn.Embedding(config.vocab_size, config.n_embd),
            drop=nn.Dropout(config.dropout),
            h=nn.ModuleList([LlamaBlock(config) for _ in range(config.n_layer)]),
            ln_f=RMSNorm(config.n_embd, eps=cfg_get(config, "rmsnorm_eps", 1e-5)),
        ))
        self.lm_head = nn.Linear(config.n_embd, config.vocab_size, bias=False)
        self.transformer.wte.weight = self.lm_head.weight
        scheme, std = cfg_get(config, "init_scheme", "KarpathyGPT2"), cfg_get(config, "init_std", 0.02)
        self.apply(lambda m: init_module_weights(m, scheme, std))
        for name, p in self.named_parameters():
            if name.endswith("c_proj.weight"):
                nn.init.normal_(p, mean=0.0, std=0.02 / math.sqrt(2 * config.n_layer))

    @staticmethod
    def get_tp_plan():
        return {"attn.c_attn": "colwise", "attn.c_proj": "rowwise", "mlp.w1": "colwise", "mlp.w2": "colwise",
                "mlp.c_proj": "rowwise"}

    def get_num_params(self, non_embedding=True, exclude_embeddings=False):
        n = sum(p.numel() for p in self.parameters())
        if exclude_embeddings:
            n -= self.transformer.wte.weight.numel()
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
        for i, block in enumerate(self.transformer.h):
            if ckpt and self.training and i % cfg_get(cfg, "checkpoint_every_n", 1) == 0:
                x, extra = _checkpoint(block, x, freqs, use_reentrant=False)
            else:
                x, extra = block(x, freqs)
            if extra:
                router_logits.append(extra["router_logits"])
                experts.append(extra["selected_experts"])
        x = self.transformer.ln_f(x)
        aux, acc, logits, loss = {}, None, None, None
        if targets is not None:
            if get_logits:
                logits = self.lm_head(x)
                loss = F.cross_entropy(logits.view(-1, logits.size(-1)), targets.view(-1), ignore_index=-1)
            else:
                from .common import chunked_cross_entropy

                loss, _, acc = chunked_cross_entropy(x, self.lm_head.weight, targets, compute_accuracy=compute_accuracy)
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
                "router_logits": torch.stack(router_logits, 0) if router_logits else None, "accuracy": acc}
