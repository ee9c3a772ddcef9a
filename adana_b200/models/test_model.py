"""`--model test`: the smallest RoPE + GELU decoder, weight-only LayerNorm with eps = `--rmsnorm_eps` (named RMSNorm2
upstream), a bias-free 4x GELU MLP whose first matrix is called `w1`, token embedding always tied to the head,
full-logit cross entropy.  Kept for quick experiments, with the reference's parameter names
(src/models/test.py:1-238)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.rope import precompute_freqs_cis
from .common import BaseLM, LayerNorm, cfg_get, init_module_weights
from .llama import LlamaAttention


class TestMLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.w1 = nn.Linear(config.n_embd, 4 * config.n_embd, bias=False)
        self.c_proj = nn.Linear(4 * config.n_embd, config.n_embd, bias=False)

    def forward(self, x):
        return self.c_proj(F.gelu(self.w1(x))), {}


class TestBlock(nn.Module):
    def __init__(self, config):
        super().__init__()
        eps = cfg_get(config, "rmsnorm_eps", 1e-5)
        self.ln_1 = LayerNorm(config.n_embd, bias=False, eps=eps)
        self.attn = LlamaAttention(config)
        self.ln_2 = LayerNorm(config.n_embd, bias=False, eps=eps)
        self.mlp = TestMLP(config)

    def forward(self, x, freqs_cis):
        x = x + self.attn(self.ln_1(x), freqs_cis)
        return x + self.mlp(self.ln_2(x))[0], {}


class Test(BaseLM):
    arch = "test"

    def __init__(self, config):
        super().__init__(config)
        self.head_dim = config.n_embd // config.n_head
        self.freqs_cis = precompute_freqs_cis(self.head_dim, config.sequence_length)
        self.transformer = nn.ModuleDict(dict(
            wte=nn.Embedding(config.vocab_size, config.n_embd),
            drop=nn.Dropout(config.dropout),
            h=nn.ModuleList([TestBlock(config) for _ in range(config.n_layer)]),
            ln_f=LayerNorm(config.n_embd, bias=False, eps=cfg_get(config, "rmsnorm_eps", 1e-5)),
        ))
        self.lm_head = nn.Linear(config.n_embd, config.vocab_size, bias=False)
        self.transformer.wte.weight = self.lm_head.weight      # always tied, whatever --weight_tying says
        self.apply(lambda m: init_module_weights(m, cfg_get(config, "init_scheme", "KarpathyGPT2"),
                                                 cfg_get(config, "init_std", 0.02)))

    def forward(self, idx, targets=None, get_logits=False, moe=False, compute_accuracy=False):
        b, t = idx.shape
        assert t <= self.config.sequence_length
        x = self.transformer.drop(self.transformer.wte(idx))
        freqs = self.freqs_cis.to(x.device)[:t]
        for block in self.transformer.h:
            x, _ = block(x, freqs)
        x = self.transformer.ln_f(x)
        loss, acc, logits = None, None, None
        if targets is not None:
            logits = self.lm_head(x)
            flat = logits.view(-1, logits.size(-1))
            loss = F.cross_entropy(flat, targets.view(-1), ignore_index=-1)
            if compute_accuracy:
                acc = (flat.argmax(-1) == targets.view(-1)).float().mean()
        else:
            logits = self.lm_head(x[:, [-1], :])
        return {"logits": logits if get_logits else None, "loss": loss, "aux_losses": {}, "router_logits": None,
                "accuracy": acc}
