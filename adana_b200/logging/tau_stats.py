"""Tau statistics of the Dana-Star optimizers (`--collect-tau-stats`).

At evaluation number 10·2^k (k = 0, 1, ...) every `tau` state tensor is reduced to sparse order
statistics — the ⌊1.1^j⌋-th smallest and largest values — and stored as
`<exp_dir>/tau_stats/tau_stats_iter_<iter>_<timestamp>.pkl`, next to one
`tau_stats_metadata.json` describing the run.  File names, pickle keys and the sampling grid
follow the reference (src/optim/tau_stats_collector.py:22-376) so its plotting scripts read
these files.  Works with the per-tensor optimizers (state on the parameters) and with the fused
engine optimizer (tau gathered from the flat shards).
"""
from __future__ import annotations

import json
import pickle
from datetime import datetime
from pathlib import Path
from typing import Dict, List, Tuple

import numpy as np
import torch

_META_FIELDS = {
    "model_params": ["model", "n_head", "n_layer", "n_embd", "head_dim", "qkv_dim", "mlp_hidden_dim",
                     "mlp_hidden_mult", "vocab_size", "dropout", "bias", "weight_tying", "parallel_block",
                     "normalization_layer_type", "elementwise_attn_output_gate"],
    "optimizer_params": ["lr", "delta", "kappa", "clipsnr", "weight_decay", "mk4A", "mk4B", "omega", "beta1",
                         "beta2", "wd_decaying", "wd_ts", "grad_clip"],
    "training_params": ["iterations", "iterations_to_run", "batch_size", "acc_steps", "sequence_length",
                        "eval_interval", "log_interval", "warmup_steps", "seed", "data_seed"],
    "loss_params": ["z_loss_coeff", "hoyer_loss_coeff"],
    "initialization_params": ["init_scheme", "init_std", "residual_stream_scalar"],
    "scheduler_params": ["scheduler", "div_factor", "final_div_factor", "cos_inf_steps", "wsd_final_lr_scale",
                         "wsd_fract_decay", "decay_type"],
}


def compute_tau_order_statistics(tau_vector: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """(largest, smallest) order statistics at ranks ⌊1.1^k⌋, k = 0.., de-duplicated."""
    n = len(tau_vector)
    if n == 0:
        return np.array([]), np.array([])
    asc = np.sort(tau_vector)
    kmax = int(np.ceil(np.log(n) / np.log(1.1)))
    idx = np.unique(np.int32(1.1 ** np.arange(kmax + 1)) - 1)
    idx = np.minimum(idx, n - 1)
    return asc[(n - 1) - idx], asc[idx]


def _plain(v):
    return v.item() if isinstance(v, (np.integer, np.floating)) else v


class TauStatsCollector:
    def __init__(self, exp_dir: Path, cfg, param_names: List[str]):
        self.exp_dir = Path(exp_dir)
        self.cfg = cfg
        self.param_names = param_names
        self.tau_stats_dir = self.exp_dir / "tau_stats"
        self.tau_stats_dir.mkdir(parents=True, exist_ok=True)
        self.eval_step_counter = 0
        limit = cfg.iterations // cfg.eval_interval + 10
        self.collection_eval_steps = []
        k = 0
        while 10 * 2 ** k <= limit:
            self.collection_eval_steps.append(10 * 2 ** k)
            k += 1
        self.next_collection_idx = 0
        print(f"[TauStats] Will collect at eval steps: {self.collection_eval_steps[:10]}... in {self.tau_stats_dir}")
        self._save_metadata()

    def should_collect(self, curr_iter: int, is_eval_step: bool) -> bool:
        if not is_eval_step:
            return False
        self.eval_step_counter += 1
        if self.next_collection_idx >= len(self.collection_eval_steps):
            return False
        if self.eval_step_counter == self.collection_eval_steps[self.next_collection_idx]:
            self.next_collection_idx += 1
            return True
        return False

    def _tau_tensors(self, opt) -> Dict[str, torch.Tensor]:
        eng = getattr(opt, "engine", None)
        if eng is not None:
            return eng.full_param_dict("tau")
        out = {}
        for group in opt.param_groups:
            names = group.get("param_names", [])
            for i, p in enumerate(group["params"]):
                st = opt.state.get(p)
                if st and "tau" in st:
                    out[names[i] if i < len(names) else f"param_group_{id(group)}_idx_{i}"] = st["tau"]
        return out

    def collect(self, opt, curr_iter: int):
        print(f"[TauStats] Collecting at iteration {curr_iter} (eval step {self.eval_step_counter})")
        stats = {}
        for name, tau in self._tau_tensors(opt).items():
            flat = tau.detach().float().cpu().flatten().numpy()
            largest, smallest = compute_tau_order_statistics(flat)
            stats[name] = {"shape": tuple(tau.shape), "largest_order_stats": largest,
                           "smallest_order_stats": smallest, "num_elements": len(flat)}
        if not stats:
            print("[TauStats] Warning: No tau statistics found in optimizer state")
            return
        stamp = datetime.now().strftime("%Y%m%d_%H%M%S")
        path = self.tau_stats_dir / f"tau_stats_iter_{curr_iter:08d}_{stamp}.pkl"
        with open(path, "wb") as f:
            pickle.dump({"metadata": {"timestamp": stamp, "iteration": curr_iter,
                                      "eval_step_number": self.eval_step_counter},
                         "tau_statistics": stats}, f)
        print(f"[TauStats] Saved {len(stats)} parameter tau statistics to: {path}")

    def _save_metadata(self):
        cfg = self.cfg
        arch = cfg.model + (f"_heads{cfg.n_head}" if hasattr(cfg, "n_head") else "")
        meta = {"timestamp": datetime.now().strftime("%Y%m%d_%H%M%S"), "optimizer": cfg.opt, "architecture": arch,
                "collection_schedule": self.collection_eval_steps}
        for section, fields in _META_FIELDS.items():
            meta[section] = {f: _plain(getattr(cfg, f)) for f in fields if hasattr(cfg, f)}
        if hasattr(cfg, "no_qknorm"):
            meta["model_params"]["qk_normalization"] = not cfg.no_qknorm
        with open(self.tau_stats_dir / "tau_stats_metadata.json", "w") as f:
            json.dump(meta, f, indent=2, default=str)
