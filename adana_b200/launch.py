"""Experiment launcher: `python -m adana_b200.launch --arch enoki --opt dana-star-mk4 --heads 36 --nproc 8
--distributed_backend fsdp ...`.

One front-end for what the reference does in `scripts/launch.sh` (flags :62-99, derivations :136-254,
launch :351-380): it turns (architecture, optimizer, heads) into a full `adana_b200.main` command line —
model shape and peak LR from the scaling rules, Chinchilla iteration count `20·params / tokens_per_step`,
warm-up `iters/50`, weight-decay time scale `iters/10`, the per-optimizer weight-decay convention
(log-time family: `wd = ω / wd_ts` with `--wd_decaying`; everything else: `wd = ω / (lr · iters)`), the
`cos_inf` schedule that ends at 10 % of the peak — and starts one process per GPU with torchrun on
127.0.0.1.  Unknown flags are forwarded to the trainer.  `--dry` prints the command instead of running.
`plan()` returns the derived configuration so that sweep / restart / benchmark drivers
(`adana_b200/experiments.py`) and tests can use it without spawning anything.
"""
from __future__ import annotations

import argparse
import math
import os
import shlex
import subprocess
import sys
from dataclasses import dataclass, field
from typing import List

from .config.scaling import compute_dimensions, compute_lr

LOGTIME = ("adana", "dana-mk4", "dana-star", "dana-star-mk4")


def _parser():
    p = argparse.ArgumentParser(allow_abbrev=False, description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    p.add_argument("--arch", required=True, choices=["enoki", "qwen3"])
    p.add_argument("--opt", required=True)
    p.add_argument("--heads", required=True, type=int)
    p.add_argument("--nproc", type=int, default=1)
    p.add_argument("--batch_size", type=int, default=32)
    p.add_argument("--acc_steps", type=int, default=1)
    p.add_argument("--seq_len", type=int, default=2048)
    p.add_argument("--kappa", type=float, default=0.85)
    p.add_argument("--clipsnr", type=float, default=2.0)
    p.add_argument("--omega", type=float, default=4.0)
    p.add_argument("--delta", type=float, default=8.0)
    p.add_argument("--gamma_3_factor", type=float, default=1.0)
    p.add_argument("--wd_ts_divisor", type=float, default=None)
    p.add_argument("--wd_ts_const", type=float, default=None)
    p.add_argument("--lr", type=float, default=None)
    p.add_argument("--iterations", type=int, default=None)
    p.add_argument("--warmup_steps", type=int, default=None)
    p.add_argument("--grad_clip", type=float, default=0.5)
    p.add_argument("--init_scheme", default="ScaledGPT")
    p.add_argument("--n_layer", type=int, default=None, help="override the scaling rule's depth")
    p.add_argument("--no_compile", action="store_true")
    p.add_argument("--no_wandb", action="store_true")
    p.add_argument("--wandb_offline", action="store_true")
    p.add_argument("--wandb_group", default=None)
    p.add_argument("--eval_interval", type=int, default=115)
    p.add_argument("--log_interval", type=int, default=50)
    p.add_argument("--latest_ckpt_interval", type=int, default=1000)
    p.add_argument("--permanent_ckpt_interval", type=int, default=0)
    p.add_argument("--distributed_backend", default="nccl")
    p.add_argument("--no_auto_resume", action="store_true")
    p.add_argument("--iterations_to_run", type=int, default=None)
    p.add_argument("--z_loss_coeff", type=float, default=None)
    p.add_argument("--scheduler", default="cos_inf")
    p.add_argument("--dataset", default="fineweb_100")
    p.add_argument("--master_port", type=int, default=0)
    p.add_argument("--dry", action="store_true")
    return p


@dataclass
class Plan:
    argv: List[str]
    env: dict = field(default_factory=dict)
    summary: dict = field(default_factory=dict)

    def torchrun(self, nproc: int, port: int) -> List[str]:
        return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
                "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "adana_b200.main", *self.argv]


def plan(a, extra: List[str]) -> Plan:
    dims = compute_dimensions(a.arch, a.heads)
    if a.n_layer is not None:
        dims["n_layer"] = a.n_layer
        dims["non_emb_params"] = 12 * dims["n_embd"] ** 2 * a.n_layer
        dims["total_params"] = dims["non_emb_params"] + 2 * dims["n_embd"] * 50304
    global_batch = a.batch_size * a.acc_steps
    lr = a.lr if a.lr is not None else compute_lr(a.arch, a.opt, dims["non_emb_params"], kappa=a.kappa,
                                                  batch_size=global_batch)
    if lr is None:
        raise SystemExit(f"ERROR: No LR formula found for optimizer '{a.opt}' in scaling rules. Please provide --lr explicitly.")
    tokens_per_step = a.batch_size * a.acc_steps * a.seq_len
    iters = a.iterations if a.iterations is not None else int(20 * dims["total_params"] / tokens_per_step)
    warmup = a.warmup_steps if a.warmup_steps is not None else int(iters / 50)
    if a.wd_ts_const is not None and a.wd_ts_divisor is not None:
        raise SystemExit("ERROR: Cannot specify both --wd_ts_divisor and --wd_ts_const")
    wd_ts = a.wd_ts_const if a.wd_ts_const is not None else int(iters / (a.wd_ts_divisor or 10))
    wd_ts = max(wd_ts, 1)
    logtime_flags = ["--delta", a.delta, "--kappa", a.kappa, "--gamma_3_factor", a.gamma_3_factor]
    decaying = ["--wd_decaying", "--wd_ts", wd_ts]
    if a.opt in LOGTIME:
        wd = a.omega / wd_ts
        opt = ["--opt", a.opt, *logtime_flags, *(["--clipsnr", a.clipsnr] if a.opt.endswith("mk4") else []), *decaying]
    elif a.opt == "adamw":
        wd, opt = a.omega / (lr * iters), ["--opt", "adamw", "--beta1", 0.9, "--beta2", 0.999]
    elif a.opt == "ademamix":
        wd = a.omega / (lr * iters)
        opt = ["--opt", "ademamix", "--beta1", 0.9, "--beta2", 0.999, *logtime_flags, "--adema_beta3_warmup", iters,
               "--adema_alpha_warmup", iters]
    elif a.opt == "adamw-decaying-wd":
        wd, opt = a.omega / wd_ts, ["--opt", a.opt, "--beta1", 0.9, "--beta2", 0.999, *decaying]
    elif a.opt == "ademamix-decaying-wd":
        wd = a.omega / wd_ts
        opt = ["--opt", a.opt, "--beta1", 0.9, "--beta2", 0.999, *logtime_flags, "--adema_beta3_warmup", iters,
               "--adema_alpha_warmup", iters, *decaying]
    elif a.opt == "d-muon":
        wd = a.omega / (lr * iters)
        opt = ["--opt", "d-muon", "--beta1", 0.8, "--beta2", 0.999, "--momentum", 0.95, "--nesterov", "True",
               "--muon_ns_steps", 5]
    elif a.opt == "manau":
        wd = a.omega / (lr * iters)
        opt = ["--opt", "manau", "--delta", a.delta, "--kappa", a.kappa, "--clipsnr", a.clipsnr, "--momentum", 0.95,
               "--nesterov", "True", "--muon_ns_steps", 5, "--matched_adamw_rms", 0.2, "--mk4A", 0.0, "--mk4B", 0.0,
               "--wd_decaying", "--wd_ts", int(iters)]
    else:
        wd, opt = a.omega / (lr * iters), ["--opt", a.opt]
    arch = ["--weight_tying", "False"]
    if a.arch == "qwen3":
        arch += ["--elementwise_attn_output_gate", "--normalization_layer_type", "rmsnorm"]
    sched = ["--scheduler", a.scheduler]
    if a.scheduler == "cos_inf":
        sched += ["--cos_inf_steps", 0, "--div_factor", 1e2, "--final_div_factor", 1e-1]
    argv = ["--model", a.arch, "--n_head", dims["n_head"], "--n_layer", dims["n_layer"], "--n_embd", dims["n_embd"],
            "--qkv_dim", dims["qkv_dim"], "--mlp_hidden_dim", dims["mlp_hidden_dim"], "--sequence_length", a.seq_len,
            "--batch_size", a.batch_size, "--acc_steps", a.acc_steps, "--lr", lr, "--weight_decay", wd,
            "--iterations", iters, "--warmup_steps", warmup, "--grad_clip", a.grad_clip, "--init-scheme", a.init_scheme,
            "--dataset", a.dataset, "--distributed_backend", a.distributed_backend, "--eval_interval", a.eval_interval,
            "--log_interval", a.log_interval, "--latest_ckpt_interval", a.latest_ckpt_interval,
            "--permanent_ckpt_interval", a.permanent_ckpt_interval, *opt, *arch, *sched]
    if not a.no_compile:
        argv.append("--compile")
    if not a.no_wandb:
        argv += ["--wandb", "--wandb_project", os.environ.get("WANDB_PROJECT", "my-project")]
        if os.environ.get("WANDB_ENTITY"):
            argv += ["--wandb_entity", os.environ["WANDB_ENTITY"]]
    if not a.no_auto_resume:
        argv.append("--auto_resume")
    if a.iterations_to_run is not None:
        argv += ["--iterations_to_run", a.iterations_to_run]
    # passed explicitly, as the reference's launcher does (scripts/launch.sh:351-369), whatever the parser defaults are
    argv += ["--config_format", "base", "--dropout", 0.0, "--seed", 0,
             "--z_loss_coeff", a.z_loss_coeff if a.z_loss_coeff is not None else os.environ.get("Z_LOSS_COEFF", "1e-4")]
    if a.wandb_group:
        argv += ["--wandb_group", a.wandb_group, "--run_prefix", a.wandb_group]
    for key in ("DATASETS_DIR", "RESULTS_BASE_FOLDER"):
        if os.environ.get(key):
            argv += ["--" + key.lower(), os.environ[key]]
    argv = [str(x) for x in argv] + list(extra)
    env = {"PYTORCH_CUDA_ALLOC_CONF": os.environ.get("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")}
    if a.wandb_offline:
        env["WANDB_MODE"] = "offline"
    summary = dict(arch=a.arch, opt=a.opt, heads=a.heads, **{k: dims[k] for k in ("n_embd", "n_head", "n_layer",
                   "mlp_hidden_dim", "qkv_dim", "non_emb_params", "total_params")}, lr=lr, weight_decay=wd, wd_ts=wd_ts,
                   iterations=iters, warmup_steps=warmup, tokens_per_step=tokens_per_step, nproc=a.nproc,
                   backend=a.distributed_backend)
    return Plan(argv=argv, env=env, summary=summary)


def banner(s: dict, a) -> str:
    lines = ["=" * 60, "Training Launch", "=" * 60,
             f"Architecture: {s['arch']}", f"Optimizer:    {s['opt']}", f"Heads:        {s['heads']}",
             f"Dimensions:   n_embd={s['n_embd']}, n_head={s['n_head']}, n_layer={s['n_layer']}",
             f"MLP hidden:   {s['mlp_hidden_dim']}", f"QKV dim:      {s['qkv_dim']}",
             f"Parameters:   non_emb={s['non_emb_params']} ({s['non_emb_params'] / 1e6:.1f}M), total={s['total_params']} "
             f"({s['total_params'] / 1e6:.1f}M)",
             f"LR:           {s['lr']}", f"Weight Decay: {s['weight_decay']} (omega={a.omega}, wd_ts={s['wd_ts']})",
             f"Iterations:   {s['iterations']} (from 20 * total_params / tokens_per_step)",
             f"Warmup:       {s['warmup_steps']} (iterations/50)", f"Scheduler:    {a.scheduler}",
             f"Grad clip:    {a.grad_clip}",
             f"Batch:        {a.batch_size}x{a.acc_steps}x{a.seq_len} ({a.nproc} GPUs, global={a.batch_size * a.acc_steps})",
             f"Dataset:      {a.dataset}", f"Backend:      {s['backend']}", "=" * 60]
    return "\n".join(lines)


def main(argv=None) -> int:
    a, extra = _parser().parse_known_args(argv)
    pl = plan(a, extra)
    print(banner(pl.summary, a))
    single = a.distributed_backend in ("single",) and a.nproc == 1
    port = a.master_port or (29500 + os.getpid() % 2000)
    cmd = [sys.executable, "-m", "adana_b200.main", *pl.argv] if single else pl.torchrun(a.nproc, port)
    print(" ".join(shlex.quote(c) for c in cmd))
    if a.dry:
        return 0
    return subprocess.call(cmd, env={**os.environ, **pl.env})


if __name__ == "__main__":
    raise SystemExit(main())
