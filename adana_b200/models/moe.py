"""Mixture-of-experts layers and router losses.

`MoE` (token choice, top-k, optional always-on shared experts) and `ExpertChoiceMoE` (each expert
picks its top-c tokens) keep the reference's semantics and module names (`experts.{i}`, `router`;
src/models/moe.py:131-244) but dispatch differently: token→expert assignments are sorted once and
each expert runs on one contiguous slice of the permuted activations (a grouped-GEMM-shaped
schedule) instead of one boolean-mask gather per expert.  Router losses: entropy regulariser,
Switch-Transformer load balancing, router z-loss (src/models/moe.py:14-128).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


def log_mean(x, dim):
    return torch.logsumexp(x, dim=dim) - math.log(x.shape[dim])


def entropy_reg(logits, mean_over_batch: bool = True):
    logp = F.log_softmax(logits, dim=-1)
    if mean_over_batch:
        logp = log_mean(logp, 0)
    return (logp * logp.exp()).sum(-1).mean()      # minus the entropy


def load_balancing_loss(logits, expert_indices):
    """num_experts * mean_e( fraction of tokens routed to e * mean router probability of e )."""
    n_exp = logits.shape[1]
    hit = F.one_hot(expert_indices, n_exp).amax(dim=-2)
    frac = hit.float().mean(dim=0)
    prob = torch.exp(log_mean(F.log_softmax(logits, dim=-1), dim=0))
    return (frac * prob).float().mean() * n_exp


def router_z_loss(router_logits):
    return (torch.logsumexp(router_logits, dim=-1) ** 2).float().sum() / router_logits.shape[0]


def router_losses(cfg, logits, selected, eval_mode=False):
    if eval_mode:
        return {"moe_entropy_loss": entropy_reg(logits), "moe_aux_loss": load_balancing_loss(logits, selected),
                "moe_z_loss": router_z_loss(logits)}
    kind = cfg.moe_router_loss
    if kind == "entropy":
        return {"moe_entropy_loss": entropy_reg(logits)}
    if kind == "load_balancing_only":
        return {"moe_aux_loss": load_balancing_loss(logits, selected)}
    if kind == "load_balancing_z_loss":
        return {"moe_aux_loss": load_balancing_loss(logits, selected), "moe_z_loss": router_z_loss(logits)}
    return {}


def _route(router_logits, top_k, order):
    if order == "softmax_topk":
        probs = F.softmax(router_logits, dim=1, dtype=torch.float32)
        return torch.topk(probs, top_k)
    if order == "topk_softmax":
        w, sel = torch.topk(router_logits, top_k)
        return F.softmax(w, dim=-1, dtype=torch.float32), sel
    raise ValueError(f"Unknown softmax_order: {order}")


def grouped_expert_apply(x, experts, selected, weights):
    """sum_k weights[t,k] * experts[selected[t,k]](x[t]) with one contiguous slice per expert."""
    T, k = selected.shape
    flat_e = selected.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    tok = (order // k)
    counts = torch.bincount(flat_e, minlength=len(experts)).tolist()
    xs = x[tok]
    out = torch.zeros_like(x)
    ws = weights.reshape(-1)[order].to(x.dtype)
    start = 0
    for e, n in enumerate(counts):
        if n == 0:
            continue
        y, _ = experts[e](xs[start:start + n])
        out.index_add_(0, tok[start:start + n], y * ws[start:start + n, None])
        start += n
    return out


class MoE(nn.Module):
    def __init__(self, config, mlp):
        super().__init__()
        assert config.moe_num_experts > 0
        self.experts = nn.ModuleList([mlp(config=config) for _ in range(config.moe_num_experts)])
        self.n_shared_experts = config.moe_num_shared_experts
        self.router = nn.Linear(config.n_embd, config.moe_num_experts - self.n_shared_experts, bias=False)
        self.top_k = config.moe_num_experts_per_tok
        self.softmax_order = config.moe_softmax_order

    def forward(self, inputs):
        x = inputs.view(-1, inputs.shape[-1])
        logits = self.router(x)
        weights, selected = _route(logits, self.top_k, self.softmax_order)
        out = grouped_expert_apply(x, self.experts[self.n_shared_experts:], selected, weights)
        for e in self.experts[:self.n_shared_experts]:
            out = out + e(x)[0]
        return out.view_as(inputs), {"router_logits": logits, "selected_experts": selected}


class ExpertChoiceMoE(nn.Module):
    def __init__(self, config, mlp):
        super().__init__()
        assert config.moe_num_experts > 0
        self.n_experts = config.moe_num_experts
        self.experts = nn.ModuleList([mlp(config=config) for _ in range(config.moe_num_experts)])
        self.router = nn.Linear(config.n_embd, config.moe_num_experts, bias=False)
        self.capacity_factor = config.capacity_factor
        self.softmax_order = config.moe_softmax_order
        self.top_k = int(self.capacity_factor * config.batch_size * config.sequence_length / config.moe_num_experts)

    def forward(self, inputs):
        x = inputs.view(-1, inputs.shape[-1])
        top_k = max(1, min(self.top_k, int(self.capacity_factor * x.shape[0] / self.n_experts)))
        logits = self.router(x)
        if self.softmax_order == "softmax_topk":
            weights, chosen = torch.topk(F.softmax(logits, dim=1, dtype=torch.float32).T, top_k)
        elif self.softmax_order == "topk_softmax":
            weights, chosen = torch.topk(logits.T, top_k)
            weights = F.softmax(weights, dim=0, dtype=torch.float32)
        else:
            raise ValueError(f"Unknown softmax_order: {self.softmax_order}")
        out = torch.zeros_like(x)
        for i, expert in enumerate(self.experts):
            y, _ = expert(x[chosen[i]])
            out.index_add_(0, chosen[i], y * weights[i, :, None].to(x.dtype))
        return out.view_as(inputs), {"router_logits": logits, "selected_experts": chosen}
