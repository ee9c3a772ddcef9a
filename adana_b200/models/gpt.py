"""GPT-2 style base model (`--model base`): learned positions, fused QKV, GELU MLP (4x), pre-LN
blocks (optionally parallel attention+MLP), optional weight tying, dense→MoE checkpoint upcycling.
Parameter names follow the reference (src/models/base.py:36-609): transformer.{wte,wpe,h.{i},ln_f},
lm_head; blocks hold ln_1, attn.{c_attn,c_proj}, ln_2, mlp.{c_fc,c_proj}.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint as _checkpoint

from .common import BaseLM, LayerNorm, cfg_get, depth_scaled_init_, init_module_weights


class CausalSelfAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        assert config.n_embd % config.n_head == 0
        self.c_attn = nn.Linear(config.n_embd, 3 * config.n_embd, bias=config.bias)
        self.c_proj = nn.Linear(config.n_embd, config.n_embd, bias=config.bias)
        self.resid_dropout = nn.Dropout(config.dropout)
        self.n_head, self.dropout = config.n_head, config.dropout

    def forward(self, x):
        B, T, C = x.shape
        hd = C // self.n_head
        q, k, v = (t.view(B, T, -1, hd).transpose(1, 2) for t in self.c_attn(x).chunk(3, dim=-1))
        y = F.scaled_dot_product_attention(q, k, v, attn_mask=None, is_causal=True,
                                           dropout_p=self.dropout if self.training else 0.0)
        return self.resid_dropout(self.c_proj(y.transpose(1, 2).contiguous().view(B, T, -1)))


class MLP(nn.Module):
    def __init__(self, config, exp_factor=1.0):
        super().__init__()
        hidden = int(exp_factor * 4 * config.n_embd)
        self.c_fc = nn.Linear(config.n_embd, hidden, bias=config.bias)
        self.c_proj = nn.Linear(hidden, config.n_embd, bias=config.bias)
        self.dropout = nn.Dropout(config.dropout)
        self.activation = nn.GELU()

    def forward(self, x):
        return self.dropout(self.c_proj(self.activation(self.c_fc(x)))), {}


class Block(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.ln_1 = LayerNorm(config.n_embd, bias=config.bias)
        self.attn = CausalSelfAttention(config)
        self.parallel = cfg_get(config, "parallel_block", False)
        if not self.parallel:
            self.ln_2 = LayerNorm(config.n_embd, bias=config.bias)
        if cfg_get(config, "moe", False):
            from .moe import ExpertChoiceMoE, MoE

            routing = config.moe_routing
            if routing == "standard_gating":
                self.mlp = MoE(config, MLP)
            elif routing == "expert_choice":
                self.mlp = ExpertChoiceMoE(config, MLP)
            else:
                raise ValueError(f"Unknown routing: {routing}")
        else:
            self.mlp = MLP(config, cfg_get(config, "mlp_dim_exp_factor", 1.0))
        self.scale = cfg_get(config, "residual_stream_scalar", 1.0)

    def forward(self, x):
        if self.parallel:
            h = self.ln_1(x)
            y, extra = self.mlp(h)
            return x + self.scale * (self.attn(h) + y), extra
        x = x + self.scale * self.attn(self.ln_1(x))
        y, extra = self.mlp(self.ln_2(x))
        return x + self.scale * y, extra


class GPTBase(BaseLM):
    arch = "base"

    def __init__(self, config):
        super().__init__(config)
        self.transformer = nn.ModuleDict(dict(
            wte=nn.Embedding(config.vocab_size, config.n_embd),
            wpe=nn.Embedding(config.sequence_length, config.n_embd),
            drop=nn.Dropout(config.dropout),
            h=nn.ModuleList([Block(config) for _ in range(config.n_layer)]),
            ln_f=LayerNorm(config.n_embd, bias=config.bias),
        ))
        self.lm_head = nn.Linear(config.n_embd, config.vocab_size, bias=False)
        if config.weight_tying:
            self.transformer.wte.weight = self.lm_head.weight
        scheme, std = cfg_get(config, "init_scheme", "KarpathyGPT2"), cfg_get(config, "init_std", 0.02)
        self.apply(lambda m: init_module_weights(m, scheme, std))
        if scheme == "KarpathyGPT2":
            depth_scaled_init_(self.named_parameters(), ("c_proj.weight",), scheme, std, config.n_layer)
        for name, p in self.named_parameters():
            if name.endswith("router.weight"):   # routers start row-normalised with the same spread
                with torch.no_grad():
                    dim = 1 if cfg_get(config, "moe_routing", "standard_gating") == "standard_gating" else 0
                    s = p.std()
                    p.div_(p.sum(dim=dim, keepdim=True))
                    p.mul_(s / p.std())

    @staticmethod
    def get_tp_plan():
        return {"attn.c_attn": "colwise", "attn.c_proj": "rowwise", "mlp.c_fc": "colwise", "mlp.c_proj": "rowwise"}

    def forward(self, idx, targets=None, get_logits=False, moe=False, compute_accuracy=False):
        cfg = self.config
        b, t = idx.shape
        assert t <= cfg.sequence_length, \
            f"Cannot forward sequence of length {t}, block size is only {cfg.sequence_length}"
        pos = torch.arange(0, t, dtype=torch.long, device=idx.device).unsqueeze(0)
        tok_emb = self.transformer.wte(idx)
        x = self.transformer.drop(tok_emb + self.transformer.wpe(pos))
        router_logits, experts = [], []
        ckpt = cfg_get(cfg, "activation_checkpointing", False)
        every = cfg_get(cfg, "checkpoint_every_n", 1)
        for i, block in enumerate(self.transformer.h):
            if ckpt and self.training and i % every == 0:
                x, extra = _checkpoint(block, x, use_reentrant=False)
            else:
                x, extra = block(x)
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
            hoyer = self.compute_hoyer_loss(tok_emb)
            aux["hoyer_loss"] = hoyer
            loss = loss + cfg_get(cfg, "hoyer_loss_coeff", 0.0) * hoyer
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

    # ---- checkpoint interop ---------------------------------------------------------------------------
    def load_dense_into_moe(self, dense_state: dict):
        """Upcycle a dense checkpoint: every expert starts from the dense MLP, the router stays as initialised."""
        own = self.state_dict()
        out = {}
        for k, v in own.items():
            if k in dense_state:
                out[k] = dense_state[k]
            elif ".mlp.experts." in k:
                parts = k.split(".")
                i = parts.index("experts")
                out[k] = dense_state[".".join(parts[:i] + parts[i + 2:])]
            else:
                out[k] = v
        self.load_state_dict(out)

    @classmethod
    def from_pretrained(cls, config, state_dict):
        model = cls(config)
        sd = {k.replace("_orig_mod.", "").replace("module.", ""): v for k, v in state_dict.items()}
        if cfg_get(config, "moe", False) and not any(".experts." in k for k in sd):
            model.load_dense_into_moe(sd)
        else:
            model.load_state_dict(sd)
        return model
