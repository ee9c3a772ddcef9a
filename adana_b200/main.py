"""Training entry point: `python -m adana_b200.main --model enoki --opt dana-star-mk4 ...`
(one process per GPU under `torchrun` for the `ddp`/`nccl`/`gloo`/`fsdp` backends).

Flow (behaviour parity with the reference's src/main.py:262-493): backend → per-rank
batch/seed adjustment → seeds → experiment name/dir (+ resume) → data readers → model →
`backend.transform_model` (attaches the kernel engine) → named parameter groups → optimizer →
scheduler → `train()` → `summary.json`.
"""
from __future__ import annotations

import argparse
import copy
import hashlib
import json
import os
import random
import sys
from pathlib import Path

import numpy as np
import torch

from . import config, distributed
from .config.scaling import apply_scaling_rule
from .data import DataReader, MultiFileDataReader, get_dataset
from .models.utils import get_model
from .optim.muon import CombinedScheduler
from .optim.registry import build_optimizer
from .optim.schedule import build_scheduler
from .train.checkpoint import checkpoint_exists
from .train.loop import train

EXP_NAME_IGNORE = ["eval_interval", "full_eval_at", "distributed_backend", "latest_ckpt_interval",
                   "permanent_ckpt_interval", "wandb", "wandb_project", "wandb_entity", "wandb_group",
                   "results_base_folder", "run_prefix", "wandb_run_prefix", "plot_router_logits", "auto_resume",
                   "resume_from", "device", "seed", "resume_from_swa", "datasets_dir", "iterations_to_run",
                   "async_checkpoint", "device_timing", "nvtx", "heartbeat_timeout",
                   # not flags of the reference's parser: a value derived in get_args, and the switch that only makes
                   # the initial weights those of the reference (same directory as the reference's run)
                   "adema_alpha", "init_compat"]


def get_args(argv=None):
    parser = argparse.ArgumentParser(allow_abbrev=False)
    parser.add_argument("--config_format", default="base", choices=config.registered_formats())
    pre, rest = parser.parse_known_args(argv)
    args = config.parse_args_with_format(format=pre.config_format, base_parser=parser, args=rest, namespace=pre)
    apply_scaling_rule(args)
    if getattr(args, "tp_size", 1) > 1:
        if args.distributed_backend != "fsdp":
            raise ValueError("--tp_size > 1 requires --distributed_backend fsdp")
        if getattr(args, "moe", False):
            raise ValueError("--tp_size > 1 is not supported with --moe")
    if args.adema_beta3 is None:
        args.adema_beta3 = 1.0 - args.delta / args.iterations
    if getattr(args, "adema_alpha", None) is None:
        args.adema_alpha = args.iterations ** (1.0 - args.kappa)
    return args, parser


def get_exp_name(args, parser, distributed_backend=None, key_args=("model", "dataset", "opt"),
                 ignore_args=EXP_NAME_IGNORE):
    """`[prefix_]{B}x{acc}_model-.._dataset-.._opt-..__k-v...` of the non-default flags; names over
    200 characters collapse to an md5 tag."""
    defaults = vars(parser.parse_args([]))
    head = []
    for k in key_args:
        if hasattr(args, k):
            v = getattr(args, k)
            if k == "model" and getattr(args, "moe", False):
                v = f"moe_{v}"
            head.append(f"{k}-{v}")
    prefix = f"{args.batch_size}x{args.acc_steps}_" + "_".join(head)
    if args.run_prefix is not None:
        prefix = f"{args.run_prefix}_{prefix}"
    from .config.flags import REFERENCE_FLAG_ORDER

    # the reference's flags in the reference's order, then the flags that exist only here
    rank_of = {k: i for i, k in enumerate(REFERENCE_FLAG_ORDER)}
    keys = sorted(vars(args), key=lambda k: rank_of.get(k, len(rank_of)))      # stable: extras keep their own order
    tail = [f"{k}-{getattr(args, k)}" for k in keys
            if k not in ignore_args and k in defaults and k not in key_args and getattr(args, k) != defaults[k]]
    name = f"{prefix}__{'_'.join(tail)}" if tail else prefix
    if len(name) > 200:
        name = f"{prefix}__hash_{hashlib.md5(name.encode()).hexdigest()[:8]}"
        print(f"Warning: Experiment name too long, using hash: {name}")
    return name


def get_data_readers(args, verbose=True):
    data = get_dataset(args)
    val_src = data["val"]
    common = dict(local_batch_size=args.batch_size, sequence_length=args.sequence_length, seed=args.data_seed,
                  with_replacement=False)
    train_keys = sorted(k for k in data if k.startswith("train_"))
    if "train" in data and not train_keys:
        train_reader = DataReader(data_src=data["train"], auto_shard=True, keep_in_ram=args.data_in_ram, **common)
    elif train_keys:
        train_reader = MultiFileDataReader(data_files={k: data[k] for k in train_keys}, auto_shard=True,
                                           keep_in_ram=True, **common)
    else:
        raise ValueError("No train data found in dataset")
    # every rank evaluates the same validation batches
    val_reader = DataReader(data_src=val_src, auto_shard=False, keep_in_ram=True, **common)
    if verbose:
        print(f"Num training tokens: {train_reader.num_tokens} \nNum validation tokens: {val_reader.num_tokens}")
    return {"train": train_reader, "val": val_reader}


def named_param_groups(model, backend):
    """The model's decay / no-decay name lists resolved to tensors, keeping the names in each group."""
    raw = backend.get_raw_model(model)
    specs = raw.get_parameter_group_specs()
    by_name = dict(model.named_parameters())
    n_opt = 0
    for g in specs:
        params, names = [], []
        for p_name in g["params"]:
            for t in backend.translate_model_parameter_name_for_node(p_name):
                params.append(by_name[t])
                names.append(t)
        g["params"], g["param_names"] = params, names
        n_opt += sum(p.numel() for p in params)
    return specs, n_opt


def main(args, parser):
    backend = distributed.make_backend_from_args(args)
    args = backend.get_adjusted_args_for_process(args)
    args.world_size = backend.get_world_size()
    if args.full_eval_at is None:
        args.full_eval_at = []
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True
    torch.manual_seed(args.seed)
    random.seed(args.seed)
    np.random.seed(args.seed)
    if "cuda" in args.device:
        torch.cuda.set_device(torch.device(args.device))

    exp_name = args.experiment_name or get_exp_name(args, parser, backend)
    exp_dir = Path(args.results_base_folder) / exp_name
    if args.resume_from is not None:
        r = Path(args.resume_from)
        r = r.parent if r.suffix == ".pt" else r
        exp_dir = r.parent.parent if r.parent.name == "ckpts" else r
        exp_name = exp_dir.name
    master = backend.is_master_process()
    if master and args.wandb:
        args.renorm_weight_decay = args.weight_decay * args.lr * args.iterations
        _init_wandb(args, exp_name, exp_dir)
    if master:
        print(f"Starting Experiment: {exp_name}\nExperiment Directory: {exp_dir}\nConfig:\n{vars(args)}\n")
        print(f"Loading dataset: '{args.dataset}'")
    readers = get_data_readers(args, verbose=master)

    model = get_model(args).to(args.device)
    if master:
        print(f"\nModel:\n{model}")
    raw = backend.get_raw_model(model)
    counts = (raw.get_num_params(), raw.get_num_params(exclude_embeddings=True), raw.get_num_params(non_embedding=False))
    model = backend.transform_model(model)
    specs, n_opt = named_param_groups(model, backend)
    if master:
        print("number of parameters: %.2fM" % (counts[0] / 1e6,))
        print("number of non-embedding parameters: %.2fM" % (counts[1] / 1e6,))
        print("number of parameters (with all embeddings): %.2fM" % (counts[2] / 1e6,))
        print("number of optimized parameters: %.2fM" % ((n_opt if backend.engine is None else backend.engine.num_params()) / 1e6,))
    backend.param_counts = (counts[0], n_opt if backend.engine is None else backend.engine.num_params())

    opt = build_optimizer(args, model, specs, engine=backend.engine)
    backend.engine_optimizer = hasattr(opt, "engine")
    if master:
        print(f"\nOptimizer:\n{opt}")
    scheduler = None
    if args.scheduler != "none":
        assert args.warmup_steps < args.iterations, "Warmup steps must be < iterations."
        scheduler = CombinedScheduler(opt, args) if args.opt == "muon" else build_scheduler(args, opt)

    if args.resume_from is None:
        # rank 0 looks and tells the others: a slower rank that looked for itself could find the checkpoint that
        # rank 0 has meanwhile begun to write at iteration 0
        found = [checkpoint_exists(exp_dir / "ckpts" / "latest")]
        if torch.distributed.is_available() and torch.distributed.is_initialized() and torch.distributed.get_world_size() > 1:
            torch.distributed.broadcast_object_list(found, src=0)
        if found[0]:
            if not args.auto_resume:
                raise ValueError(f"The experiment dir {exp_dir} already exists. To resume training, set "
                                 "auto_resume=True. Otherwise, specify a different experiment name. ")
            args.resume_from = str(exp_dir / "ckpts" / "latest")
        elif master:
            exp_dir.mkdir(parents=True, exist_ok=True)

    stats = train(model=model, opt=opt, datareaders=readers, scheduler=scheduler, exp_dir=exp_dir,
                  distributed_backend=backend, cfg=args)
    stats["args"] = {k: v for k, v in vars(args).items() if _jsonable(v)}
    if master:
        exp_dir.mkdir(parents=True, exist_ok=True)
        with open(exp_dir / "summary.json", "w") as f:
            json.dump(stats, f)
    setattr(readers["train"], "disable_coordination", True)
    backend.finalize()
    return stats


def _jsonable(v):
    try:
        json.dumps(v)
        return True
    except (TypeError, ValueError):
        return False


def _init_wandb(args, exp_name, exp_dir):
    try:
        import wandb
    except ImportError:
        print("wandb is not installed; continuing without it")
        args.wandb = False
        return
    run_id = None
    id_file = exp_dir / "wandb_run_id.txt"
    resuming = args.resume_from is not None or (args.auto_resume and checkpoint_exists(exp_dir / "ckpts" / "latest"))
    if resuming and id_file.exists():
        run_id = id_file.read_text().strip()
    # The run is named after the experiment directory (`--wandb_run_prefix` is parsed and ignored, as in the reference,
    # whose plotting scripts look runs up by this name), keeps its files inside that directory, and plots the training
    # and validation metrics against "iter" (src/main.py:322-338).
    wandb.init(project=args.wandb_project, entity=args.wandb_entity, group=args.wandb_group, name=exp_name,
               config=copy.copy(vars(args)), id=run_id or None, resume="allow" if run_id else None, dir=str(exp_dir))
    wandb.define_metric("iter")
    for pattern in ("train/*", "val/*", "lr"):
        wandb.define_metric(pattern, step_metric="iter")


def cli(argv=None):
    args, parser = get_args(argv)
    return main(args, parser)


if __name__ == "__main__":
    cli()
