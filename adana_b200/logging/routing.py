"""MoE routing summaries for wandb (expert selection frequencies for three layers)."""
from __future__ import annotations

import torch


def visualize_routing(router_logits, cfg):
    """router_logits [batches, layers, tokens, experts] -> dict of scalars (+ a histogram)."""
    logs = {}
    try:
        import wandb

        logs["router/logits"] = wandb.Histogram(router_logits.float().flatten().cpu().numpy())
    except Exception:
        pass
    L, E, k = cfg.n_layer, cfg.moe_num_experts, cfg.moe_num_experts_per_tok
    for layer in sorted({0, L // 2, L - 1}):
        sel = torch.topk(router_logits[:, layer], k, dim=-1).indices
        hit = torch.nn.functional.one_hot(sel, E).amax(dim=-2).float().mean(dim=(0, 1))
        for i in range(E):
            logs[f"router/layer_{layer}_expert_{i}_selection"] = hit[i].item()
    return logs
