"""Shared model pieces: norms, initialisation schemes, the LM base class and the loss head.

`BaseLM` gives every architecture the reference's model contract
(src/models/base.py:165-609): `forward(idx, targets=None, get_logits=False, moe=False,
compute_accuracy=False) -> {logits, loss, aux_losses, router_logits, accuracy}`,
`get_parameter_group_specs()` (decay = Linear weights, no-decay = biases, norms,
embeddings; names sorted inside each group), `get_num_params`, `generate`,
`generate_from_string`, `crop_sequence_length`.

Two execution paths share one set of `nn.Parameter`s:
  * the PyTorch path in each model's `forward` (autograd; CPU oracle and fallback), and
  * the kernel path of `adana_b200.runtime.engine` (manual forward/backward over the
    sm_100a ops), selected when an engine is attached to the model.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


class LayerNorm(nn.Module):
    """LayerNorm with an optional bias (weight-only by default), eps 1e-5."""

    def __init__(self, ndim: int, bias: bool = False, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(ndim))
        self.bias = nn.Parameter(torch.zeros(ndim)) if bias else None
        self.eps = eps

    def forward(self, x):
        return F.layer_norm(x, self.weight.shape, self.weight, self.bias, self.eps)


class RMSNorm(nn.Module):
    """x / sqrt(mean(x^2) + eps) computed in fp32, cast back, times weight."""

    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        xf = x.float()
        out = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).type_as(x)
        return out * self.weight


NORM_MODULES = (LayerNorm, RMSNorm, nn.LayerNorm, nn.Embedding)


def make_norm(kind: str, dim: int, bias: bool = False, eps: float = 1e-5) -> nn.Module:
    return RMSNorm(dim, eps) if kind == "rmsnorm" else LayerNorm(dim, bias, eps)


def init_module_weights(module: nn.Module, scheme: str, init_std: float) -> None:
    """KarpathyGPT2: N(0, init_std); Standard: linear 1/sqrt(fan_in), embeddings N(0,1);
    ScaledGPT: linear 1/sqrt(fan_in), embeddings 1/sqrt(d)."""
    if isinstance(module, nn.Linear):
        std = 1.0 / math.sqrt(module.weight.size(1)) if scheme in ("Standard", "ScaledGPT") else init_std
        nn.init.normal_(module.weight, mean=0.0, std=std)
        if module.bias is not None:
            nn.init.zeros_(module.bias)
    elif isinstance(module, nn.Embedding):
        if scheme == "Standard":
            std = 1.0
        elif scheme == "ScaledGPT":
            std = 1.0 / math.sqrt(module.weight.size(1))
        else:
            std = init_std
        nn.init.normal_(module.weight, mean=0.0, std=std)


def depth_scaled_init_(named_params, suffixes, scheme: str, init_std: float, n_layer: int) -> None:
    """Residual-output projections get a 1/sqrt(2L) smaller std (KarpathyGPT2, ScaledGPT)."""
    for name, p in named_params:
        if not name.endswith(suffixes):
            continue
        if scheme == "KarpathyGPT2":
            nn.init.normal_(p, mean=0.0, std=init_std / math.sqrt(2 * n_layer))
        elif scheme == "ScaledGPT":
            nn.init.normal_(p, mean=0.0, std=1.0 / math.sqrt(2 * p.size(1) * n_layer))


def chunked_cross_entropy(hidden, weight, targets, chunk_size=256, z_loss_coeff=0.0,
                          compute_z_loss=False, compute_accuracy=False):
    """lm_head + CE in chunks of `chunk_size` positions (PyTorch path).

    Returns (ce_mean + z_coeff * z_mean, z_mean | None, accuracy | None); means are over all
    B*T positions, `ignore_index = -1` (behaviour parity: reference
    src/models/chunked_loss.py:68-151).
    """
    B, T, _ = hidden.shape
    ce = hidden.new_zeros((), dtype=torch.float32)
    zs = hidden.new_zeros((), dtype=torch.float32)
    correct = 0
    for s in range(0, T, chunk_size):
        logits = F.linear(hidden[:, s:s + chunk_size], weight)
        flat = logits.reshape(-1, logits.size(-1))
        tgt = targets[:, s:s + chunk_size].reshape(-1)
        ce = ce + F.cross_entropy(flat, tgt, ignore_index=-1, reduction="sum")
        if compute_z_loss:
            zs = zs + torch.logsumexp(flat, dim=-1).pow(2).sum()
        if compute_accuracy:
            correct = correct + (flat.argmax(-1) == tgt).sum()
    n = B * T
    loss = ce / n
    z_mean = zs / n if compute_z_loss else None
    if z_mean is not None:
        loss = loss + z_loss_coeff * z_mean
    acc = (correct / n).float() if compute_accuracy else None
    return loss, z_mean, acc


class _ByteTokenizer:
    """Fallback when the GPT-2 BPE files are unavailable offline: bytes as tokens."""

    eot_token = 50256

    def encode(self, s, allowed_special=None):
        return list(s.encode("utf-8"))

    encode_ordinary = encode

    def decode(self, ids):
        return bytes(int(i) % 256 for i in ids).decode("utf-8", errors="replace")


def get_tokenizer():
    try:
        import tiktoken

        return tiktoken.get_encoding("gpt2")
    except Exception:
        return _ByteTokenizer()


class BaseLM(nn.Module):
    """Common behaviour of all language models in this package."""

    decay_module_types = (nn.Linear,)

    def __init__(self, config):
        super().__init__()
        assert config.vocab_size is not None and config.sequence_length is not None
        self.config = config
        self._tokenizer = None
        self._engine = None  # set by adana_b200.runtime.engine.attach()

    # ---- tokenizer is created lazily: constructing a model never needs the network ----
    @property
    def tokenizer(self):
        if self._tokenizer is None:
            self._tokenizer = get_tokenizer()
        return self._tokenizer

    # ---- parameter bookkeeping -------------------------------------------------------------------
    def get_num_params(self, non_embedding=True, exclude_embeddings=False):
        n = sum(p.numel() for p in self.parameters())
        wpe = getattr(self.transformer, "wpe", None) if hasattr(self, "transformer") else None
        if non_embedding and wpe is not None:
            n -= wpe.weight.numel()
        if exclude_embeddings:
            n -= self.transformer.wte.weight.numel()
            if not self.config.weight_tying:
                n -= self.lm_head.weight.numel()
        return n

    def get_parameter_group_specs(self):
        decay, no_decay = set(), set()
        for mn, m in self.named_modules():
            for pn, _ in m.named_parameters(recurse=False):
                full = f"{mn}.{pn}" if mn else pn
                if pn.endswith("bias"):
                    no_decay.add(full)
                elif pn.endswith("weight") and isinstance(m, self.decay_module_types):
                    decay.add(full)
                else:
                    no_decay.add(full)
        if self.config.weight_tying and "lm_head.weight" in decay:
            decay.discard("lm_head.weight")
        names = {n for n, _ in self.named_parameters()}
        decay &= names
        no_decay &= names
        assert not (decay & no_decay), f"parameters in both groups: {decay & no_decay}"
        assert not (names - (decay | no_decay)), f"parameters in no group: {names - (decay | no_decay)}"
        return [{"params": sorted(decay)}, {"params": sorted(no_decay), "weight_decay": 0.0}]

    def crop_sequence_length(self, sequence_length):
        assert sequence_length <= self.config.sequence_length
        self.config.sequence_length = sequence_length
        wpe = getattr(self.transformer, "wpe", None)
        if wpe is not None:
            wpe.weight = nn.Parameter(wpe.weight[:sequence_length])

    # ---- auxiliary losses --------------------------------------------------------------------------
    @staticmethod
    def compute_hoyer_loss(emb):
        """mean over tokens of ||x||_1 / (||x||_2 + 1e-8)."""
        return (emb.abs().sum(-1) / (emb.norm(p=2, dim=-1) + 1e-8)).mean()

    @staticmethod
    def compute_z_loss(logits):
        return torch.logsumexp(logits, dim=-1).pow(2).mean()

    def _loss_head(self, x, tok_emb, targets, get_logits, compute_accuracy):
        """Shared tail of the PyTorch path: ln_f output -> loss dict pieces."""
        cfg = self.config
        aux, acc, logits = {}, None, None
        z_coeff = getattr(cfg, "z_loss_coeff", 0.0)
        if get_logits:
            logits = self.lm_head(x)
            flat = logits.view(-1, logits.size(-1))
            loss = F.cross_entropy(flat, targets.view(-1), ignore_index=-1)
            z = self.compute_z_loss(flat)
            loss = loss + z_coeff * z
        else:
            loss, z, acc = chunked_cross_entropy(x, self.lm_head.weight, targets, compute_z_loss=True,
                                                 z_loss_coeff=z_coeff, compute_accuracy=compute_accuracy)
        aux["z_loss"] = z
        hoyer = self.compute_hoyer_loss(tok_emb)
        aux["hoyer_loss"] = hoyer
        loss = loss + getattr(cfg, "hoyer_loss_coeff", 0.0) * hoyer
        return loss, logits, aux, acc

    # ---- sampling --------------------------------------------------------------------------------------
    @torch.no_grad()
    def generate(self, idx, max_new_tokens, temperature=1.0, top_k=None):
        for _ in range(max_new_tokens):
            ctx = idx if idx.size(1) <= self.config.sequence_length else idx[:, -self.config.sequence_length:]
            logits = self(ctx, get_logits=True)["logits"][:, -1, :] / temperature
            if top_k is not None:
                kth = torch.topk(logits, min(top_k, logits.size(-1))).values[:, [-1]]
                logits = logits.masked_fill(logits < kth, float("-inf"))
            nxt = torch.multinomial(F.softmax(logits.float(), dim=-1), num_samples=1)
            idx = torch.cat((idx, nxt), dim=1)
        return idx

    @torch.no_grad()
    def generate_from_string(self, in_str, max_new_tokens, temperature=1.0, top_k=None):
        dev = next(self.parameters()).device
        ids = self.tokenizer.encode(in_str, allowed_special={"<|endoftext|>"})
        idx = torch.tensor(ids, dtype=torch.long, device=dev).view(1, -1)
        out = self.generate(idx, max_new_tokens, temperature, top_k).view(-1).cpu().numpy()
        return self.tokenizer.decode(out)


def cfg_get(config, name, default=None):
    v = getattr(config, name, default)
    return default if v is None else v
