"""Experiment orchestration on top of `adana_b200.launch`: grid sweeps, self-resubmitting restart jobs
and the batch-size / memory benchmark.  One module with three sub-commands replaces the reference's shell
drivers (`scripts/sweep.sh`, `scripts/restart_{enoki,qwen3}.sh`, `scripts/benchmark_batch.sh`,
`scripts/config.sh`, `scripts/cluster_list*.sh`):

    python -m adana_b200.experiments sweep   --arch enoki --opt adana --heads 8 12 --lr_mult 0.5 1 2 [--slurm] [--dry]
    python -m adana_b200.experiments restart --arch enoki --opt dana-star-mk4 --heads 16 --iterations_to_run 2000 ...
    python -m adana_b200.experiments benchmark-batch --heads 28 36 --batch 4 8 16 --nproc 4
    python -m adana_b200.experiments jobs            # squeue one-liner for this user

* sweep: every (heads x LR multiplier) point becomes one launch (or one `sbatch --wrap` of the restart
  driver under `--slurm`), all in one wandb group; the base LR comes from the scaling rules.
* restart: runs the launcher with `--auto_resume`; when the run exits cleanly because
  `--iterations_to_run` was reached and the final iteration has not been, it starts (or, under SLURM,
  `sbatch`es) itself again with RESTART_COUNT+1 — a job that fits in a scheduler slot and continues
  from the `latest` checkpoint.
* benchmark-batch: 5-iteration runs over heads x tp x batch in increasing batch order, stopping a (heads, tp) pair
  at its first out-of-memory failure; records the `[Memory] ... peak_allocated=` line and the last `iter_dt=`,
  prints and files the largest batch that fits.
Environment (`config.sh` equivalent): `ADANA_CONFIG` may name a file of KEY=VALUE lines (WANDB_*,
DATASETS_DIR, RESULTS_BASE_FOLDER, TIKTOKEN_CACHE_DIR, HF_HOME) that is loaded into the environment.
"""
from __future__ import annotations

import argparse
import itertools
import json
import os
import re
import shlex
import subprocess
import sys
from pathlib import Path

from . import launch as L
from .config.scaling import compute_dimensions, compute_lr


def load_user_config(path=None) -> dict:
    path = path or os.environ.get("ADANA_CONFIG")
    loaded = {}
    if path and Path(path).exists():
        for line in Path(path).read_text().splitlines():
            line = line.split("#", 1)[0].strip()
            if line.startswith("export "):
                line = line[len("export "):]
            if "=" in line:
                k, v = line.split("=", 1)
                loaded[k.strip()] = v.strip().strip('"').strip("'")
    os.environ.update({k: v for k, v in loaded.items() if k not in os.environ})
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    return loaded


def _launch_cmd(args_list):
    return [sys.executable, "-m", "adana_b200.launch", *[str(a) for a in args_list]]


def _sbatch(cmd, job_name, nproc, time, mem, account=None, dry=False, export=None, nodes=1):
    """Prints the `sbatch --wrap` line and, unless `dry`, submits it.  `export` adds variables to the job's environment
    on top of the submitting one (`--export=ALL,K=V`)."""
    sb = ["sbatch", f"--job-name={job_name}", f"--gres=gpu:{nproc}", f"--time={time}", f"--mem={mem}", f"--nodes={nodes}",
          f"--cpus-per-task={8 * int(nproc) if str(nproc).isdigit() else 8}"]
    if account:
        sb.append(f"--account={account}")
    if export:
        sb.append("--export=ALL," + ",".join(f"{k}={v}" for k, v in export.items()))
    sb += ["--wrap", " ".join(shlex.quote(c) for c in cmd)]
    print(" ".join(shlex.quote(c) for c in sb))
    return 0 if dry else subprocess.call(sb)


# ---- sweep ------------------------------------------------------------------------------------------------------
def cmd_sweep(a, extra):
    points = []
    for heads in a.heads:
        dims = compute_dimensions(a.arch, heads)
        # the learning-rate law at its default batch, as the reference's sweep does (scripts/sweep.sh:131-146): the sweep
        # passes --lr explicitly, so the launcher's own batch-dependent table is not consulted
        base_lr = compute_lr(a.arch, a.opt, dims["non_emb_params"], kappa=a.kappa)
        if base_lr is None:
            raise SystemExit(f"no LR law for {a.opt}; pass --base_lr")
        base_lr = a.base_lr or base_lr
        tokens = a.batch_size * a.acc_steps * 2048
        print(f"--- heads={heads} (non_emb={dims['non_emb_params'] / 1e6:.1f}M total={dims['total_params'] / 1e6:.1f}M "
              f"iters={int(20 * dims['total_params'] / tokens)}, base_lr={base_lr:.6e}) ---")
        for mult in a.lr_mult:
            largs = ["--arch", a.arch, "--opt", a.opt, "--heads", heads, "--nproc", a.nproc, "--batch_size", a.batch_size,
                     "--acc_steps", a.acc_steps, "--kappa", a.kappa, "--clipsnr", a.clipsnr, "--gamma_3_factor",
                     a.gamma_3_factor, "--lr", f"{mult * base_lr:.6e}", "--scheduler", a.scheduler,
                     "--distributed_backend", a.distributed_backend, "--wandb_group", a.wandb_group,
                     "--eval_batches", a.eval_batches]
            if a.tp_size > 1:
                largs += ["--tp_size", a.tp_size]
            if a.liger_loss:
                largs += ["--liger_loss"]
            largs += ["--z_loss_coeff", a.z_loss_coeff]
            if not a.auto_resume:
                largs += ["--no_auto_resume"]
            if a.iterations:
                largs += ["--iterations", a.iterations]
            if a.iterations_to_run:
                largs += ["--iterations_to_run", a.iterations_to_run]
            if a.wandb_offline:
                largs += ["--wandb_offline"]
            if a.wd_ts_const is not None:
                largs += ["--wd_ts_const", a.wd_ts_const]
            elif a.wd_ts_divisor is not None:
                largs += ["--wd_ts_divisor", a.wd_ts_divisor]
            largs += extra
            points.append((heads, mult, largs))
    rc = 0
    for heads, mult, largs in points:
        name = f"{a.arch}-{a.opt}-h{heads}-lr{mult}"
        if a.slurm:
            cmd = [sys.executable, "-m", "adana_b200.experiments", "restart", *[str(x) for x in largs]]
            rc |= _sbatch(cmd, name, a.nproc, a.time, a.mem, a.account, dry=a.dry)
        else:
            cmd = _launch_cmd(largs + (["--dry"] if a.dry else []))
            print(" ".join(shlex.quote(c) for c in cmd))
            rc |= subprocess.call(cmd)
    print(f"{len(points)} job(s) {'printed' if a.dry else 'submitted'}")
    return rc


# ---- restart -----------------------------------------------------------------------------------------------------
def cmd_restart(a, extra):
    count = int(os.environ.get("RESTART_COUNT", "0"))
    print(f"[restart] attempt {count}")
    largs = list(extra)
    if "--no_auto_resume" in largs:
        largs.remove("--no_auto_resume")
    rc = subprocess.call(_launch_cmd(largs))
    if rc != 0:
        print(f"[restart] launch exited with {rc}; not resubmitting")
        return rc
    if "--iterations_to_run" not in largs or count + 1 >= a.max_restarts:
        return 0
    if a.finished_marker and Path(a.finished_marker).exists():      # e.g. the experiment's summary.json: the run is complete
        print(f"[restart] {a.finished_marker} exists; not resubmitting")
        return 0
    env = {**os.environ, "RESTART_COUNT": str(count + 1)}
    me = [sys.executable, "-m", "adana_b200.experiments", "restart", "--max_restarts", str(a.max_restarts),
          *(["--finished_marker", a.finished_marker] if a.finished_marker else []), *largs]
    if os.environ.get("SLURM_JOB_ID"):
        # resubmit with the resources of the running job (scripts/restart_enoki.sh:46-94): account, time limit, nodes,
        # GPUs per node, memory (0 = all of the node's, must be kept) and name; the restart count travels with --export
        info = subprocess.run(["scontrol", "show", "job", os.environ["SLURM_JOB_ID"]], capture_output=True, text=True).stdout

        def field(name, default):
            m = re.search(rf"\b{name}=(\S+)", info)
            return m.group(1) if m else default

        gpus = os.environ.get("SLURM_GPUS_PER_NODE")
        if not gpus:
            m = re.search(r"gres/gpu[:=](\S+)", info) or re.search(r"gpu[:=](\d+)", info)
            gpus = m.group(1) if m else 1
        return _sbatch(me, field("JobName", os.environ.get("SLURM_JOB_NAME", "adana-restart")), gpus,
                       field("TimeLimit", "4:00:00"), field("MinMemoryNode", os.environ.get("SLURM_MEM_PER_NODE", "0")),
                       field("Account", os.environ.get("SLURM_JOB_ACCOUNT")), export={"RESTART_COUNT": count + 1},
                       nodes=field("NumNodes", 1))
    return subprocess.call(me, env=env)


# ---- batch-size / memory benchmark --------------------------------------------------------------------------------
def parse_run_log(text: str) -> dict:
    """Pull the facts the benchmark records out of a trainer log."""
    oom = bool(re.search(r"out of memory|OutOfMemoryError|CUDA error: out of memory", text, re.I))
    mem = re.findall(r"peak_allocated=([0-9.]+) GiB", text)
    dts = re.findall(r"iter_dt=([0-9.eE+-]+)s", text)
    return {"oom": oom, "peak_allocated_gib": float(mem[-1]) if mem else None, "iter_dt": float(dts[-1]) if dts else None}


def cmd_benchmark_batch(a, extra):
    """Largest batch that fits, per (heads, tp): 5-iteration runs in increasing batch order, stopping at the first one
    that runs out of memory (scripts/benchmark_batch.sh:57-208).  As there, `--batch` is the batch of one step over
    all data-parallel ranks (acc_steps 1): the backend divides it by world / tp."""
    results, lines = [], ["# heads  tp  batch  peak_mem(GiB)  iter_dt(s)  status"]
    for heads, tp in itertools.product(a.heads, a.tp):
        best = 0
        for batch in a.batch:
            largs = ["--arch", a.arch, "--opt", a.opt, "--heads", heads, "--nproc", a.nproc, "--batch_size", batch,
                     "--acc_steps", 1, "--iterations", a.iterations, "--warmup_steps", 3, "--scheduler", "cos", "--kappa", a.kappa,
                     "--clipsnr", 1.0, "--no_wandb", "--no_auto_resume", "--distributed_backend", "fsdp", "--log_interval", 1,
                     "--eval_interval", 9999, "--eval_batches", 4, "--latest_ckpt_interval", 0, "--permanent_ckpt_interval", 0,
                     "--dataset", a.dataset, *extra]
            if tp > 1:
                largs += ["--tp_size", tp]
            if a.dry:
                print(" ".join(shlex.quote(str(c)) for c in _launch_cmd(largs)))
                continue
            proc = subprocess.run(_launch_cmd(largs), capture_output=True, text=True)
            rec = {"heads": heads, "tp": tp, "batch": batch, "returncode": proc.returncode,
                   **parse_run_log(proc.stdout + proc.stderr)}
            rec["ok"] = proc.returncode == 0 and not rec["oom"]
            results.append(rec)
            print(json.dumps(rec), flush=True)
            if not rec["ok"]:
                lines.append(f"heads={heads}  tp={tp}  batch={batch}  STATUS={'OOM' if rec['oom'] else 'FAILED'}")
                break                      # a larger batch cannot fit either
            best = batch
            lines.append(f"heads={heads}  tp={tp}  batch={batch}  peak_mem={rec['peak_allocated_gib']}  iter_dt={rec['iter_dt']}  OK")
        if not a.dry:
            print(f">>> heads={heads}  tp={tp}  max_batch={best}")
            lines.append(f"heads={heads}  tp={tp}  MAX_BATCH={best}")
    if not a.dry and a.results_file:
        Path(a.results_file).parent.mkdir(parents=True, exist_ok=True)
        Path(a.results_file).write_text("\n".join(lines) + "\n")
    return 0


def cmd_jobs(a, extra):
    return subprocess.call(["squeue", "-u", os.environ.get("USER", ""), "-o", "%.10i %.40j %.8T %.10M %.6D %R"])


def main(argv=None) -> int:
    load_user_config()
    p = argparse.ArgumentParser(allow_abbrev=False)
    sub = p.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("sweep")
    s.add_argument("--arch", default="enoki")
    s.add_argument("--opt", default="adana")
    s.add_argument("--heads", type=int, nargs="+", default=[8])
    s.add_argument("--lr_mult", type=float, nargs="+", default=[1.0])
    s.add_argument("--base_lr", type=float, default=None)
    s.add_argument("--kappa", type=float, default=0.85)
    s.add_argument("--clipsnr", type=float, default=0.25)
    s.add_argument("--gamma_3_factor", type=float, default=1.0)
    s.add_argument("--wd_ts_divisor", type=float, default=10)
    s.add_argument("--wd_ts_const", type=float, default=None)
    s.add_argument("--batch_size", type=int, default=8)
    s.add_argument("--acc_steps", type=int, default=16)
    s.add_argument("--nproc", type=int, default=4)
    s.add_argument("--scheduler", default="cos_inf")
    s.add_argument("--distributed_backend", default="fsdp")
    s.add_argument("--tp_size", type=int, default=1)
    s.add_argument("--wandb_group", default="fsdp-experiment")
    s.add_argument("--iterations_to_run", type=int, default=None)
    s.add_argument("--iterations", type=int, default=None, help="instead of the Chinchilla count")
    s.add_argument("--eval_batches", type=int, default=4)
    s.add_argument("--z_loss_coeff", default="1e-4")
    s.add_argument("--liger_loss", action="store_true")
    s.add_argument("--auto_resume", action="store_true", help="resume from the latest checkpoint (default: fresh start)")
    s.add_argument("--wandb_offline", action="store_true")
    s.add_argument("--slurm", action="store_true")
    s.add_argument("--account", default=None)
    s.add_argument("--time", default="3:00:00")
    s.add_argument("--mem", default="0")
    s.add_argument("--dry", action="store_true")
    r = sub.add_parser("restart")
    r.add_argument("--max_restarts", type=int, default=50)
    r.add_argument("--finished_marker", default=None)
    b = sub.add_parser("benchmark-batch")
    b.add_argument("--arch", default="enoki")
    b.add_argument("--opt", default="dana-star-mk4")
    b.add_argument("--heads", type=int, nargs="+", default=[28, 32, 36, 44, 48])
    b.add_argument("--tp", type=int, nargs="+", default=[1, 4])
    b.add_argument("--batch", type=int, nargs="+", default=[4, 8, 16, 32])
    b.add_argument("--nproc", type=int, default=4)
    b.add_argument("--dataset", default="synthetic-zipf")
    b.add_argument("--kappa", type=float, default=0.85)
    b.add_argument("--iterations", type=int, default=5)
    b.add_argument("--results_file", default="logs/benchmark_batch_results.txt")
    b.add_argument("--dry", action="store_true")
    sub.add_parser("jobs")
    a, extra = p.parse_known_args(argv)
    return {"sweep": cmd_sweep, "restart": cmd_restart, "benchmark-batch": cmd_benchmark_batch, "jobs": cmd_jobs}[a.cmd](a, extra)


if __name__ == "__main__":
    raise SystemExit(main())
