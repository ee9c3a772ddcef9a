"""Launcher and experiment drivers: derived hyper-parameters, command construction, log parsing."""
import math

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
