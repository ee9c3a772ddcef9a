"""Launcher and experiment drivers: derived hyper-parameters, command construction, log parsing."""
import math

import pytest
from pathlib import Path

from adana_b200 import experiments, launch


def _plan(*argv):
    a, extra = launch._parser().parse_known_args(list(argv))
    return launch.plan(a, extra), a


def test_enoki_dana_star_mk4_plan_follows_the_scaling_rules():
    p, a = _plan("--arch", "enoki", "--opt", "dana-star-mk4", "--heads", "36", "--nproc", "8", "--distributed_backend", "fsdp",
                 "--batch_size", "64", "--acc_steps", "8", "--no_wandb")
    cmd = " ".join(str(x) for x in p.torchrun(a.nproc, 29500))
    # 20 tokens per parameter at 64 x 8 x 2048 tokens per step; warm-up = iterations / 50; wd_ts = iterations / 10
    assert "--iterations 37226" in cmd and "--warmup_steps 744" in cmd and "--wd_ts 3722" in cmd
    assert "--opt dana-star-mk4" in cmd and "--wd_decaying" in cmd and "--clipsnr" in cmd and "--kappa 0.85" in cmd
    assert "--nproc-per-node=8" in cmd and "--master-addr 127.0.0.1" in cmd and "--distributed_backend fsdp" in cmd
    assert "--n_embd 2304" in cmd and "--n_head 36" in cmd and "--qkv_dim 64" in cmd
    lr = float(cmd.split("--lr ")[1].split()[0])
    assert math.isclose(lr, 1.0406e-4, rel_tol=2e-3)
    wd = float(cmd.split("--weight_decay ")[1].split()[0])
    assert math.isclose(wd, 4.0 / 3722, rel_tol=1e-3)            # omega / wd_ts


def test_adamw_plan_uses_lr_dependent_weight_decay_and_qwen3_flags():
    p, a = _plan("--arch", "qwen3", "--opt", "adamw", "--heads", "16", "--nproc", "4", "--distributed_backend", "fsdp",
                 "--batch_size", "32", "--acc_steps", "4", "--no_wandb")
    cmd = " ".join(str(x) for x in p.torchrun(a.nproc, 29500))
    lr = float(cmd.split("--lr ")[1].split()[0])
    it = int(cmd.split("--iterations ")[1].split()[0])
    wd = float(cmd.split("--weight_decay ")[1].split()[0])
    assert math.isclose(wd, 4.0 / (lr * it), rel_tol=1e-6)       # omega / (lr * iterations)
    assert "--beta2 0.999" in cmd and "--elementwise_attn_output_gate" in cmd and "--normalization_layer_type rmsnorm" in cmd
    assert "--wd_decaying" not in cmd


def test_sweep_prints_one_job_per_grid_point(capsys):
    rc = experiments.main(["sweep", "--arch", "enoki", "--opt", "adana", "--heads", "8", "12", "--lr_mult", "0.5", "1", "2",
                           "--slurm", "--dry"])
    out = capsys.readouterr().out
    assert rc == 0 and out.count("sbatch ") == 6 and "6 job(s) printed" in out
    assert "experiments restart" in out and "--heads 12" in out


def test_benchmark_log_parsing():
    text = "\n".join(["iter 3", "[Memory] after iter 1 peak_allocated=52.61 GiB reserved=60 GiB",
                      "Train: Iter=5 iter_dt=1.23e+00s lr=1e-3", ""])
    rec = experiments.parse_run_log(text)
    assert rec == {"oom": False, "peak_allocated_gib": 52.61, "iter_dt": 1.23}
    assert experiments.parse_run_log("torch.OutOfMemoryError: CUDA out of memory")["oom"] is True


def test_user_config_file_is_loaded_without_overriding_the_environment(tmp_path, monkeypatch):
    import os

    f = tmp_path / "cfg"
    f.write_text("\n".join(["# comment", "export WANDB_PROJECT=proj", "DATASETS_DIR='/data/x'", "HOME=/nope", ""]))
    monkeypatch.delenv("WANDB_PROJECT", raising=False)
    monkeypatch.delenv("DATASETS_DIR", raising=False)
    monkeypatch.setenv("HOME", "/keep")
    loaded = experiments.load_user_config(str(f))
    assert loaded["WANDB_PROJECT"] == "proj" and os.environ["DATASETS_DIR"] == "/data/x" and os.environ["HOME"] == "/keep"


def test_launcher_builds_the_same_training_command_as_the_reference_launch_script(ref_src, tmp_path):
    """`scripts/launch.sh` of the reference is run with a stand-in `torchrun` that only prints its arguments; the flags
    it would hand to `main.py` (model shape, learning rate, weight decay, its time scale, iterations, warm-up, schedule,
    optimizer flags, compile / resume switches) must equal those of `python -m adana_b200.launch --dry`."""
    import itertools
    import os
    import shlex
    import shutil
    import subprocess
    import sys

    script = ref_src.parent / "scripts" / "launch.sh"
    if not script.exists() or shutil.which("bash") is None:
        pytest.skip("the reference's launch script or bash is not available")
    fake = tmp_path / "bin"
    fake.mkdir()
    (fake / "torchrun").write_text("#!/bin/bash\necho \"FAKE_TORCHRUN $@\"\n")
    (fake / "torchrun").chmod(0o755)
    env = {k: v for k, v in os.environ.items() if k not in ("DATASETS_DIR", "RESULTS_BASE_FOLDER", "WANDB_PROJECT", "WANDB_ENTITY")}
    env["PATH"] = f"{fake}:{env['PATH']}"
    root = Path(__file__).resolve().parent.parent

    def parse(tokens):
        flags, i = {}, 0
        while i < len(tokens):
            t = tokens[i]
            if t.startswith("--") and "=" in t:
                k, v = t.split("=", 1)
                flags[k] = v
                i += 1
            elif t.startswith("--") and i + 1 < len(tokens) and not tokens[i + 1].startswith("--"):
                flags[t] = tokens[i + 1]
                i += 2
            else:
                if t.startswith("--"):
                    flags[t] = True
                i += 1
        return flags

    def reference(args):
        out = subprocess.run(["bash", "scripts/launch.sh", *args], cwd=ref_src.parent, env=env, capture_output=True,
                             text=True, timeout=120).stdout
        line = [ln for ln in out.splitlines() if ln.startswith("FAKE_TORCHRUN")]
        if not line:
            assert "ERROR" in out, out[-500:]        # e.g. no learning-rate law for this optimizer and no --lr
            return None
        return parse(shlex.split(line[0])[1:])

    def ours(args):
        out = subprocess.run([sys.executable, "-m", "adana_b200.launch", *args, "--dry"], cwd=root, env=env,
                             capture_output=True, text=True, timeout=120)
        line = [ln for ln in out.stdout.splitlines() if "adana_b200.main" in ln]
        if not line:
            assert out.returncode != 0
            return None
        return parse(shlex.split(line[-1]))

    cases = [["--arch", arch, "--opt", opt, "--heads", str(heads), "--no_wandb"]
             for arch, opt, heads in itertools.product(("enoki", "qwen3"), ("adamw", "dana-mk4", "dana-star-mk4", "ademamix",
                                                                            "d-muon", "adamw-decaying-wd"), (8, 36))
             if (arch, heads) in (("enoki", 36), ("qwen3", 8))]
    cases += [["--arch", "enoki", "--opt", "dana-star-mk4", "--heads", "36", "--nproc", "8", "--distributed_backend", "fsdp",
               "--batch_size", "64", "--acc_steps", "8", "--no_wandb"],
              ["--arch", "enoki", "--opt", "adana", "--heads", "12", "--kappa", "0.8", "--omega", "2.0", "--wd_ts_const", "1000",
               "--no_wandb", "--no_compile"],
              ["--arch", "qwen3", "--opt", "dana-mk4", "--heads", "16", "--lr", "0.003", "--iterations", "5000",
               "--wd_ts_divisor", "5", "--iterations_to_run", "700", "--no_wandb"]]
    ignore = {"--datasets_dir", "--results_base_folder", "--master-addr", "--master-port", "--nnodes", "--standalone"}
    for args in cases:
        want, got = reference(args), ours(args)
        assert (want is None) == (got is None), args       # refused by both or by neither
        if want is None:
            continue
        assert want.pop("--nproc_per_node") == got.pop("--nproc-per-node", got.pop("--nproc_per_node", None))
        for key in (set(want) | set(got)) - ignore:
            a, b = want.get(key), got.get(key)
            if a == b:
                continue
            assert a is not None and b is not None and abs(float(a) - float(b)) <= 1e-12 * max(1.0, abs(float(a))), (args, key, a, b)


def test_sweep_submits_the_same_grid_as_the_reference_sweep_script(ref_src, tmp_path, capsys):
    """`scripts/sweep.sh --dry` of the reference (a copy whose configuration block is edited the way a user edits it)
    against `python -m adana_b200.experiments sweep --slurm --dry`: the same jobs in the same order, and for every job
    the same launcher arguments (optimizer, heads, processes, batch, kappa, clip-SNR, the learning rate of the grid
    point, schedule, backend, group, evaluation batches, z-loss, resume switch, weight-decay time scale)."""
    import re
    import shlex
    import shutil
    import subprocess

    src = ref_src.parent / "scripts"
    if not (src / "sweep.sh").exists() or shutil.which("bash") is None:
        pytest.skip("the reference's sweep script or bash is not available")
    work = tmp_path / "ref"
    shutil.copytree(ref_src.parent / "scripts", work / "scripts")
    (work / "src" / "config").mkdir(parents=True)
    for f in ("scaling.py", "scaling_rules.yaml"):
        shutil.copy(ref_src / "config" / f, work / "src" / "config" / f)
    text = (work / "scripts" / "sweep.sh").read_text()
    edits = {r'^OPT="adana"': 'OPT="dana-star-mk4"', r"^HEADS_LIST=\( 8 \)": "HEADS_LIST=( 8 12 )",
             r"^LR_MULTIPLIERS=\( 1.0 \)": "LR_MULTIPLIERS=( 0.5 1.0 2.0 )", r"^TP_SIZE=1": "TP_SIZE=2",
             r'^ITERATIONS_TO_RUN=""': 'ITERATIONS_TO_RUN="2000"'}
    for pat, rep in edits.items():
        text, n = re.subn(pat, rep, text, count=1, flags=re.M)
        assert n == 1, pat
    (work / "scripts" / "sweep.sh").write_text(text)
    out = subprocess.run(["bash", "scripts/sweep.sh", "--dry"], cwd=work, capture_output=True, text=True, timeout=300).stdout

    def flags(tokens):
        d, i = {}, 0
        while i < len(tokens):
            if tokens[i].startswith("--"):
                if i + 1 < len(tokens) and not tokens[i + 1].startswith("--"):
                    d[tokens[i]] = tokens[i + 1]
                    i += 2
                    continue
                d[tokens[i]] = True
            i += 1
        return d

    ref_jobs = []
    for line in out.splitlines():
        if line.strip().startswith("sbatch "):
            toks = shlex.split(line.strip())
            ref_jobs.append(flags(toks[toks.index("scripts/restart_enoki.sh") + 1:]))
    assert len(ref_jobs) == 6, out[-1500:]

    rc = experiments.main(["sweep", "--arch", "enoki", "--opt", "dana-star-mk4", "--heads", "8", "12", "--lr_mult", "0.5", "1.0", "2.0",
                           "--tp_size", "2", "--iterations_to_run", "2000", "--slurm", "--dry"])
    mine = []
    for line in capsys.readouterr().out.splitlines():
        if line.startswith("sbatch "):
            wrapped = shlex.split(shlex.split(line)[-1])
            mine.append(flags(wrapped[wrapped.index("restart") + 1:]))
    assert rc == 0 and len(mine) == 6
    for got, want in zip(mine, ref_jobs):
        assert got.pop("--arch") == "enoki"                      # the reference picks the architecture by its restart script
        assert set(got) == set(want), (sorted(got), sorted(want))
        for k, v in want.items():
            if k == "--lr":
                assert float(got[k]) == pytest.approx(float(v), rel=1e-6)
            elif isinstance(v, str) and re.fullmatch(r"[-+0-9.eE]+", v):
                assert float(got[k]) == float(v), k
            else:
                assert got[k] == v, k


def test_restart_resubmits_with_the_running_jobs_resources_and_stops_when_done(tmp_path, monkeypatch, capsys):
    """Under SLURM the restart driver asks `scontrol` for the running job's account, time limit, nodes, memory and name,
    and submits itself again with RESTART_COUNT + 1 (scripts/restart_enoki.sh:46-94).  `scontrol`, `sbatch` and the
    launcher are stand-ins; nothing is submitted anywhere."""
    import subprocess

    calls = []

    def fake_call(cmd, **kw):
        calls.append(("call", [str(c) for c in cmd], kw.get("env")))
        return 0

    def fake_run(cmd, **kw):
        calls.append(("run", list(cmd), None))
        return subprocess.CompletedProcess(cmd, 0, stdout="JobId=77 JobName=enoki_h16 Account=def-lab TimeLimit=04:00:00 NumNodes=1 "
                                           "MinMemoryNode=0 TresPerNode=gres/gpu:4", stderr="")

    monkeypatch.setattr(experiments.subprocess, "call", fake_call)
    monkeypatch.setattr(experiments.subprocess, "run", fake_run)
    monkeypatch.setenv("SLURM_JOB_ID", "77")
    monkeypatch.setenv("SLURM_GPUS_PER_NODE", "h100:4")
    monkeypatch.setenv("RESTART_COUNT", "2")
    args = ["restart", "--arch", "enoki", "--opt", "dana-star-mk4", "--heads", "16", "--iterations_to_run", "2000", "--no_auto_resume"]
    assert experiments.main(args) == 0
    launch, sbatch = calls[0][1], calls[-1][1]
    assert "adana_b200.launch" in launch and "--no_auto_resume" not in launch and "--iterations_to_run" in launch
    assert sbatch[0] == "sbatch" and "--export=ALL,RESTART_COUNT=3" in sbatch and "--account=def-lab" in sbatch
    assert {"--job-name=enoki_h16", "--time=04:00:00", "--mem=0", "--nodes=1", "--gres=gpu:h100:4"} <= set(sbatch)
    assert "experiments restart" in sbatch[-1] and "--heads 16" in sbatch[-1]
    # a launch that fails is not resubmitted
    calls.clear()
    monkeypatch.setattr(experiments.subprocess, "call", lambda cmd, **kw: calls.append(cmd) or 3)
    assert experiments.main(args) == 3 and len(calls) == 1
    # a finished run (its marker exists) is not resubmitted either; without --iterations_to_run nothing restarts
    monkeypatch.setattr(experiments.subprocess, "call", fake_call)
    done = tmp_path / "summary.json"
    done.write_text("{}")
    calls.clear()
    assert experiments.main(["restart", "--finished_marker", str(done), *args[1:]]) == 0
    assert [c[0] for c in calls] == ["call"]
    calls.clear()
    assert experiments.main(["restart", "--arch", "enoki", "--opt", "adana", "--heads", "8"]) == 0 and len(calls) == 1
    # outside SLURM the next segment starts right away with the count in its environment
    monkeypatch.delenv("SLURM_JOB_ID")
    calls.clear()
    assert experiments.main(args) == 0
    assert len(calls) == 2 and calls[1][2]["RESTART_COUNT"] == "3" and "restart" in calls[1][1]


def test_batch_benchmark_stops_a_configuration_at_its_first_oom(tmp_path, monkeypatch, capsys):
    """The batch-size benchmark with a stand-in launcher: batch 16 runs out of memory for tp 1, so 32 is not tried; the
    run parameters are the reference script's (scripts/benchmark_batch.sh:37-50, 108-136)."""
    import subprocess

    seen = []

    def fake_run(cmd, **kw):
        args = [str(c) for c in cmd]
        batch = int(args[args.index("--batch_size") + 1])
        tp = int(args[args.index("--tp_size") + 1]) if "--tp_size" in args else 1
        seen.append((tp, batch, args))
        if tp == 1 and batch >= 16:
            return subprocess.CompletedProcess(cmd, 1, stdout="torch.OutOfMemoryError: CUDA out of memory", stderr="")
        out = f"[Memory] GPU 0: peak_allocated={10.0 + batch:.2f} GiB\\nTrain: Iter=5 train_loss=9.1 iter_dt=1.25e-01s lr=1e-4"
        return subprocess.CompletedProcess(cmd, 0, stdout=out, stderr="")

    monkeypatch.setattr(experiments.subprocess, "run", fake_run)
    res = tmp_path / "logs" / "r.txt"
    assert experiments.main(["benchmark-batch", "--heads", "28", "--tp", "1", "4", "--batch", "4", "8", "16", "32", "--results_file", str(res)]) == 0
    assert [(tp, b) for tp, b, _ in seen] == [(1, 4), (1, 8), (1, 16), (4, 4), (4, 8), (4, 16), (4, 32)]
    text = res.read_text()
    assert "heads=28  tp=1  MAX_BATCH=8" in text and "heads=28  tp=4  MAX_BATCH=32" in text and "STATUS=OOM" in text
    args = seen[0][2]
    for flag, val in (("--iterations", "5"), ("--warmup_steps", "3"), ("--scheduler", "cos"), ("--clipsnr", "1.0"), ("--acc_steps", "1"),
                      ("--eval_interval", "9999"), ("--eval_batches", "4"), ("--latest_ckpt_interval", "0"), ("--distributed_backend", "fsdp")):
        assert args[args.index(flag) + 1] == val, flag
    out = capsys.readouterr().out
    assert ">>> heads=28  tp=1  max_batch=8" in out
