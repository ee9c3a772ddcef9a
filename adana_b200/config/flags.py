"""Command-line surface of the trainer.

The flag names and defaults follow the reference so that its launch lines keep working
(reference: src/config/base.py:22-429); the implementation is table-driven: every flag
is one `Flag` record, grouped, and `build_parser()` turns the table into argparse.
`--distributed_backend ddp` is accepted as an alias of `nccl` (the reference's name for
DDP on GPUs, src/distributed/__init__.py:3-9).
"""
from __future__ import annotations

import argparse
from dataclasses import dataclass
from typing import Any, Optional, Sequence

OPTIMIZERS = [
    "adamw", "sgd", "muon", "d-muon", "manau", "soap", "ademamix", "ademamix-decaying-wd",
    "lion", "sf-adamw", "sf-sgd", "signsgd", "signum", "prodigy", "sophiag", "adopt", "mars",
    "adafactor", "lamb", "adana", "dana-mk4", "dana-star", "dana-star-mk4", "adamw-decaying-wd",
]
DATASETS = [
    "wikitext", "shakespeare-char", "arxiv", "arxiv2000", "arxiv+wiki", "openwebtext2",
    "redpajama", "slimpajama", "slimpajama_chunk1", "redpajamav2", "fineweb", "finewebedu",
    "c4", "fineweb_100", "synthetic-zipf",
]
MODELS = ["base", "llama", "test", "enoki", "diloco", "qwen3", "qwen3next"]
BACKENDS = ["nccl", "ddp", "gloo", "fsdp", "single"]
DECAYS = ["linear", "cosine", "exp", "miror_cosine", "square", "sqrt"]


def str2bool(v) -> bool:
    if isinstance(v, bool):
        return v
    s = str(v).strip().lower()
    if s in ("1", "true", "t", "yes", "y", "on"):
        return True
    if s in ("0", "false", "f", "no", "n", "off"):
        return False
    raise argparse.ArgumentTypeError(f"expected a boolean, got {v!r}")


def none_or_str(v):
    return None if v is None or str(v) == "None" else str(v)


def truthy(v) -> bool:
    """argparse `type=bool` semantics of the reference: any non-empty string is True."""
    return bool(v)


@dataclass
class Flag:
    names: Sequence[str]
    default: Any = None
    type: Any = None
    choices: Optional[Sequence[Any]] = None
    action: Optional[str] = None
    nargs: Optional[str] = None
    dest: Optional[str] = None
    help: str = ""

    def add_to(self, p: argparse.ArgumentParser) -> None:
        kw: dict = {}
        if self.action:
            kw["action"] = self.action
            if self.action not in ("store_true", "store_false"):
                kw["type"] = self.type
            kw["default"] = self.default
        else:
            kw["default"] = self.default
            if self.type is not None:
                kw["type"] = self.type
        if self.choices is not None:
            kw["choices"] = list(self.choices)
        if self.nargs:
            kw["nargs"] = self.nargs
        if self.dest:
            kw["dest"] = self.dest
        if self.help:
            kw["help"] = self.help
        p.add_argument(*self.names, **kw)


def F(*names, **kw) -> Flag:
    return Flag(names=names, **kw)


def T(*names, **kw) -> Flag:
    return Flag(names=names, action="store_true", default=False, **kw)


GROUPS: dict[str, list[Flag]] = {
    "run": [
        F("--run_prefix", type=str), F("--experiment_name", type=str),
        F("--seed", default=0, type=int), F("--data_seed", default=1337, type=int),
        F("--eval_interval", default=200, type=int), F("--full_eval_at", nargs="+", type=int),
        F("--eval_batches", default=64, type=int), F("--device", default="cuda:0", type=str),
        F("--distributed_backend", default=None, type=str, choices=BACKENDS),
        F("--tp_size", default=1, type=int, help="tensor-parallel degree (needs fsdp)"),
        F("--log_interval", default=50, type=int),
    ],
    "checkpoint": [
        F("--results_base_folder", default="./exps", type=str),
        F("--permanent_ckpt_interval", default=0, type=int),
        F("--latest_ckpt_interval", default=0, type=int),
        F("--resume_from", type=str), F("--resume_from_swa", type=str),
        T("--auto_resume"),
        T("--async_checkpoint", help="flush checkpoint files from a background thread"),
    ],
    "logging": [
        T("--wandb"), F("--wandb_project", default="my-project", type=str),
        F("--wandb_run_prefix", default="none", type=str),
        F("--eval_seq_prefix", default="none", type=str),
        T("--log_dynamics"),
        F("--dynamics_logger_cfg", default=None, type=str),
        F("--wandb_entity", type=none_or_str), F("--wandb_group", type=none_or_str),
        T("--log_parameter_norms"), F("--norm_order", default=2),
        T("--collect-tau-stats", dest="collect_tau_stats"),
        T("--device_timing", help="time every step with CUDA events (max over ranks)"),
        T("--nvtx", help="emit NVTX ranges around step phases"),
    ],
    "schedule": [
        F("--scheduler", default="cos", choices=["linear", "cos", "wsd", "none", "cos_inf", "powerlaw"]),
        F("--div_factor", default=1e2, type=float), F("--final_div_factor", default=1.0, type=float),
        F("--cos_inf_steps", default=0, type=int),
        F("--iterations", default=15000, type=int), F("--iterations_to_run", type=int),
        F("--warmup_steps", default=3000, type=int), F("--lr", default=1e-3, type=float),
        F("--wsd_final_lr_scale", default=0.0, type=float), F("--wsd_fract_decay", default=0.1, type=float),
        F("--decay_type", default="linear", choices=DECAYS),
        F("--dd_second_decay_type", default="linear", choices=DECAYS),
        F("--dd_first_lr_factor", default=1e-2, type=float),
        F("--powerlaw_init_value", default=1.0, type=float),
        F("--powerlaw_saturation_value", default=0.0, type=float),
        F("--powerlaw_power", default=-0.5, type=float),
        F("--powerlaw_time_scale", default=1.0, type=float),
    ],
    "optimizer": [
        F("--opt", default="adamw", choices=OPTIMIZERS),
        F("--batch_size", default=50, type=int), F("--acc_steps", default=1, type=int),
        F("--weight_decay", default=1e-1, type=float),
        F("--beta1", default=0.9, type=float), F("--beta2", default=0.95, type=float),
        F("--grad_clip", default=1.0, type=float), F("--momentum", default=0.9, type=float),
        F("--shampoo_beta", default=-1.0, type=float),
        F("--precondition_frequency", default=10, type=int),
        F("--max_precond_dim", default=10000, type=int),
        F("--merge_dims", default=False, type=truthy), F("--precondition_1d", default=False, type=truthy),
        F("--normalize_grads", default=False, type=truthy),
        F("--soap_data_format", default="channels_first", type=str),
        F("--correct_bias", default=True, type=truthy), F("--nesterov", default=False, type=truthy),
        F("--muon_ns_steps", default=5, type=int), F("--muon_lr_factor", default=1.0, type=float),
        F("--matched_adamw_rms", default=0.2, type=float),
        F("--dana_momentum", default=False, type=truthy),
        F("--adema_beta3", type=float), F("--adema_alpha", type=float),
        F("--lr_outer", default=0.5, type=float), F("--k", default=1, type=int),
        F("--mu", default=0.9, type=float),
        F("--adema_beta3_warmup", type=int), F("--adema_alpha_warmup", type=int),
        F("--schedulefree_r", default=0.0, type=float), F("--weight_lr_power", default=2.0, type=float),
        F("--model_sharding", type=truthy), F("--dampening", default=0.0, type=float),
        F("--prodigy_beta3", type=float), F("--prodigy_decouple", default=True, type=truthy),
        F("--prodigy_use_bias_correction", default=False, type=truthy),
        F("--prodigy_safeguard_warmup", default=False, type=truthy),
        F("--prodigy_fsdp_in_use", default=False, type=truthy),
        F("--sophia_rho", default=0.04, type=float), F("--sophia_bs", default=480, type=int),
        F("--clipping_type", default="no", choices=["no", "local", "elementwise"]),
        F("--clip_eta", default=1.0, type=float),
        F("--mars_type", default="mars-adamw", choices=["mars-adamw", "mars-lion", "mars-shampoo"]),
        F("--mars_vr_gamma", default=0.025, type=float), F("--mars_is_approx", default=True, type=float),
        F("--mars_lr", default=3e-3, type=float), F("--mars_beta1", default=0.95, type=float),
        F("--mars_beta2", default=0.99, type=float),
        F("--adafactor_decay_rate", default=-0.8, type=float),
        F("--lamb_use_bias_correction", default=False, type=truthy),
        T("--sgd_sign_update"), T("--normalized"), F("--sgd_lr_scale", default=1.0, type=float),
        F("--adopt_decouple", default=True, type=truthy), F("--adopt_eps", default=1e-6, type=float),
        F("--g2", default=1e-3, type=float), F("--g3", default=1e-3, type=float),
        F("--delta", default=8.0, type=float), F("--kappa", default=1.0, type=float),
        F("--mk4A", default=0.0, type=float), F("--mk4B", default=0.0, type=float),
        F("--clipsnr", default=1.0, type=float),
        T("--weight_time"), T("--wd_decaying"), F("--wd_ts", default=1.0, type=float),
        T("--use_v_ema"), F("--v_ema_beta", default=0.999, type=float),
        F("--gamma_3_factor", default=1.0, type=float),
        F("--norm_type", default="linf", choices=["linf", "l2"]),
        T("--no_fused_optimizer", help="use the per-tensor PyTorch optimizer classes on GPU too"),
    ],
    "data": [
        F("--datasets_dir", default="./datasets/", type=str),
        F("--dataset", default="slimpajama", choices=DATASETS),
        F("--tokenizer", default="gpt2", type=str, choices=["gpt2", "mistral"]),
        F("--vocab_size", default=50304, type=int), T("--data_in_ram"),
        F("--zipf_exponent", default=1.0, type=float, help="exponent of the synthetic token stream"),
        F("--synthetic_tokens", default=8_000_000, type=int),
    ],
    "model": [
        F("--model", default="llama", choices=MODELS),
        F("--scaling_rule", default="none", type=str, choices=["enoki", "qwen3", "none"]),
        F("--heads", type=int), T("--parallel_block"),
        F("--use_pretrained", default="none", type=str), T("--from_dense"),
        F("--init_std", default=0.02, type=float),
        F("--init_compat", default="none", type=str, choices=["none", "reference"],
          help="reference: initial weights bit-identical to the reference's for the same --seed (enoki, qwen3)"),
        F("--init-scheme", "--init_scheme", dest="init_scheme", default="KarpathyGPT2", type=str,
          choices=["KarpathyGPT2", "Standard", "ScaledGPT"]),
        F("--residual-stream-scalar", "--residual_stream_scalar", dest="residual_stream_scalar",
          default=1.0, type=float),
        F("--dropout", default=0.0, type=float),
        F("--n_head", default=12, type=int), F("--n_kv_head", type=int,
                                               help="grouped-query attention: number of K/V heads"),
        F("--n_layer", default=24, type=int),
        F("--sequence_length", default=512, type=int), F("--n_embd", default=768, type=int),
        F("--qkv_dim", type=int), F("--mlp_hidden_dim", type=int),
        F("--multiple_of", default=256, type=int), F("--rmsnorm_eps", default=1e-5, type=float),
        F("--rope_theta", default=10000.0, type=float),
        F("--normalization_layer_type", default="rmsnorm", type=str, choices=["layernorm", "rmsnorm"]),
        T("--elementwise_attn_output_gate"),
        F("--dtype", default="bfloat16", type=str, choices=["float32", "float16", "bfloat16"]),
        F("--bias", default=False, type=str2bool), F("--weight_tying", default=True, type=str2bool),
        T("--no-qknorm", "--no_qknorm", dest="no_qknorm"),
        T("--compile"), T("--activation_checkpointing"),
        F("--checkpoint_every_n", default=1, type=int),
        F("--mlp_dim_exp_factor", default=1.0, type=float),
        F("--z_loss_coeff", default=1e-4, type=float), F("--hoyer_loss_coeff", default=0.0, type=float),
        T("--liger_loss", help="accepted for compatibility; the fused linear-CE kernel is always used on GPU"),
        T("--no_cuda_kernels", help="force the PyTorch reference ops (debugging / oracle runs)"),
    ],
    "moe": [
        T("--moe"),
        F("--moe_routing", default="standard_gating", type=str, choices=["standard_gating", "expert_choice"]),
        F("--moe_num_experts", default=8, type=int), F("--capacity_factor", default=2.0, type=float),
        F("--moe_num_shared_experts", default=0, type=int),
        F("--moe_router_loss", default="load_balancing_z_loss", type=str,
          choices=["entropy", "load_balancing_only", "load_balancing_z_loss"]),
        F("--moe_num_experts_per_tok", default=2, type=int),
        F("--moe_expert_capacity_factor", default=1.5, type=float),
        F("--moe_entropy_loss_factor", default=0.01, type=float),
        F("--moe_aux_loss_factor", default=0.1, type=float),
        F("--moe_z_loss_factor", default=0.01, type=float),
        F("--moe_softmax_order", default="topk_softmax", type=str, choices=["softmax_topk", "topk_softmax"]),
        T("--plot_router_logits"),
        T("--use_gated_shared_expert"), F("--shared_expert_intermediate_size", type=int),
        F("--decoder_sparse_step", default=1, type=int), F("--mlp_only_layers", type=str),
        Flag(names=("--expert_parallel",), action="store_true", default=True),
        Flag(names=("--no_expert_parallel",), action="store_false", dest="expert_parallel", default=True),
    ],
    "engine": [
        F("--fsdp_comm", default="auto", choices=["auto", "p2p", "nccl"],
          help="collective implementation of the sharded engine: own peer-memory kernels or NCCL"),
        F("--fsdp_prefetch", default=1, type=int, help="blocks gathered ahead of compute"),
        F("--reduce_dtype", default="bfloat16", choices=["bfloat16", "float32"]),
        F("--fsdp_weights", default="resident", choices=["resident", "gathered"],
          help="resident: every rank keeps the bf16 weights, refreshed by the optimizer step; gathered (Enoki, bf16, "
               "peer-memory plane): every rank keeps only its row slices and the GEMMs fetch weight tiles from the owners"),
        F("--attention", default="auto", choices=["auto", "native", "sdpa"],
          help="attention implementation: hand-written tcgen05 kernels or the PyTorch SDPA library call"),
        F("--heartbeat_timeout", default=0.0, type=float,
          help="seconds without a peer heartbeat before a rank aborts (0 = watchdog off)"),
    ],
}


def build_parser(base: Optional[argparse.ArgumentParser] = None) -> argparse.ArgumentParser:
    p = base or argparse.ArgumentParser(allow_abbrev=False)
    for group, flags in GROUPS.items():
        g = p.add_argument_group(group)
        for f in flags:
            f.add_to(g)
    return p


def defaults() -> argparse.Namespace:
    """Namespace holding every default (used by tests and by programmatic callers)."""
    return build_parser().parse_args([])


def parse_args(base_parser: argparse.ArgumentParser, args, namespace=None):
    parser = build_parser(base_parser)
    ns = parser.parse_args(args, namespace)
    if ns.distributed_backend == "ddp":
        ns.distributed_backend = "nccl"
    if ns.full_eval_at is None:
        ns.full_eval_at = []
    return ns


# The order in which the reference's parser defines its flags (src/config/base.py:22-429).  Experiment directory
# names list the non-default flags in this order (src/main.py:590-600), so a run started there and resumed here, or
# the other way round, looks for the same directory; flags that exist only here follow in table order.
REFERENCE_FLAG_ORDER = """
    run_prefix experiment_name seed data_seed eval_interval full_eval_at eval_batches device distributed_backend
    tp_size log_interval results_base_folder permanent_ckpt_interval latest_ckpt_interval resume_from
    resume_from_swa auto_resume wandb wandb_project wandb_run_prefix eval_seq_prefix log_dynamics
    dynamics_logger_cfg wandb_entity wandb_group log_parameter_norms norm_order scheduler div_factor
    final_div_factor cos_inf_steps iterations iterations_to_run warmup_steps lr wsd_final_lr_scale
    wsd_fract_decay decay_type dd_second_decay_type dd_first_lr_factor powerlaw_init_value
    powerlaw_saturation_value powerlaw_power powerlaw_time_scale opt batch_size acc_steps weight_decay beta1
    beta2 grad_clip momentum shampoo_beta precondition_frequency max_precond_dim merge_dims precondition_1d
    normalize_grads soap_data_format correct_bias nesterov muon_ns_steps muon_lr_factor matched_adamw_rms
    dana_momentum adema_beta3 lr_outer k mu adema_beta3_warmup adema_alpha_warmup schedulefree_r weight_lr_power
    model_sharding dampening prodigy_beta3 prodigy_decouple prodigy_use_bias_correction prodigy_safeguard_warmup
    prodigy_fsdp_in_use sophia_rho sophia_bs clipping_type clip_eta mars_type mars_vr_gamma mars_is_approx
    mars_lr mars_beta1 mars_beta2 adafactor_decay_rate lamb_use_bias_correction sgd_sign_update normalized
    sgd_lr_scale adopt_decouple adopt_eps g2 g3 delta kappa mk4A mk4B clipsnr weight_time wd_decaying wd_ts
    use_v_ema v_ema_beta gamma_3_factor norm_type collect_tau_stats datasets_dir dataset tokenizer vocab_size
    data_in_ram model scaling_rule heads parallel_block use_pretrained from_dense init_std init_scheme
    residual_stream_scalar dropout n_head n_layer sequence_length n_embd qkv_dim mlp_hidden_dim multiple_of
    rmsnorm_eps normalization_layer_type elementwise_attn_output_gate dtype bias weight_tying no_qknorm compile
    activation_checkpointing checkpoint_every_n mlp_dim_exp_factor moe moe_routing moe_num_experts
    capacity_factor moe_num_shared_experts moe_router_loss moe_num_experts_per_tok moe_expert_capacity_factor
    moe_entropy_loss_factor moe_aux_loss_factor moe_z_loss_factor moe_softmax_order plot_router_logits
    z_loss_coeff hoyer_loss_coeff liger_loss use_gated_shared_expert shared_expert_intermediate_size
    decoder_sparse_step mlp_only_layers expert_parallel
""".split()
