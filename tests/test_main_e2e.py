"""The command-line training path end to end on CPU: data -> model -> backend -> train -> eval -> checkpoint ->
early stop (`--iterations_to_run`) -> `--auto_resume` -> summary.json / metrics.jsonl; a resumed run must land on
the same weights and losses as an uninterrupted one."""
import json
import subprocess
import sys
import time
from pathlib import Path

import pytest
import torch

from conftest import torchrun

ROOT = Path(__file__).resolve().parent.parent


def _run(results, data, extra):
    cmd = [sys.executable, "-m", "adana_b200.main", "--model", "enoki", "--n_layer", "2", "--n_head", "2", "--n_embd", "64",
           "--qkv_dim", "32", "--mlp_hidden_dim", "128", "--sequence_length", "64", "--batch_size", "4", "--acc_steps", "2",
           "--vocab_size", "512", "--dataset", "synthetic-zipf", "--datasets_dir", str(data), "--opt", "dana-star-mk4",
           "--kappa", "0.85", "--clipsnr", "2.0", "--wd_decaying", "--wd_ts", "5", "--lr", "1e-3", "--iterations", "12",
           "--warmup_steps", "2", "--scheduler", "cos_inf", "--eval_interval", "4", "--eval_batches", "2",
           "--log_interval", "2", "--latest_ckpt_interval", "5", "--results_base_folder", str(results), "--device", "cpu",
           "--dtype", "float32", "--distributed_backend", "single", "--seed", "3", *extra]
    p = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    return p.stdout


def _exp_dir(results):
    dirs = [d for d in Path(results).iterdir() if d.is_dir()]
    assert len(dirs) == 1, dirs
    return dirs[0]


@pytest.mark.timeout(900)
def test_interrupted_and_resumed_run_equals_uninterrupted_run(tmp_path):
    data = tmp_path / "data"
    out = _run(tmp_path / "a", data, ["--iterations_to_run", "7"])
    assert "iterations_to_run reached" in out
    exp = _exp_dir(tmp_path / "a")
    ck = torch.load(exp / "ckpts" / "latest" / "main.pt", map_location="cpu", weights_only=False)
    assert ck["itr"] == 7 and {"model", "optimizer", "scheduler", "itr"} <= set(ck)
    assert (exp / "ckpts" / "latest" / "worker_0.pt").exists()
    out = _run(tmp_path / "a", data, ["--auto_resume"])
    assert ">Eval: Iter=12" in out and "Iter=2 " not in out.split("Resum")[-1]      # continued, did not start over
    summary = json.loads((exp / "summary.json").read_text())
    assert summary["args"]["iterations"] == 12 and "val_loss" in summary
    rows = [json.loads(l) for l in (exp / "metrics.jsonl").read_text().splitlines()]
    iters = [r["iter"] for r in rows if "train/loss" in r]
    assert iters == sorted(iters) and iters[-1] == 12 and any("final-val/loss" in r for r in rows)

    _run(tmp_path / "b", data, [])
    exp_b = _exp_dir(tmp_path / "b")
    sb = json.loads((exp_b / "summary.json").read_text())
    assert abs(summary["val_loss"][-1] - sb["val_loss"][-1]) < 1e-6            # same final validation loss
    rows_b = [json.loads(l) for l in (exp_b / "metrics.jsonl").read_text().splitlines()]
    la = {r["iter"]: r["train/loss"] for r in rows if "train/loss" in r}
    lb = {r["iter"]: r["train/loss"] for r in rows_b if "train/loss" in r}
    for it in (8, 10, 12):
        assert abs(la[it] - lb[it]) < 1e-6, (it, la[it], lb[it])


@pytest.mark.timeout(900)
def test_two_rank_fsdp_cli_run_writes_sharded_checkpoint_and_resumes(tmp_path):
    import os
    import socket

    def launch(extra):
        cmd = [*torchrun(2), "-m", "adana_b200.main", "--model", "enoki", "--n_layer", "2",
               "--n_head", "2", "--n_embd", "64", "--qkv_dim", "32", "--mlp_hidden_dim", "128", "--sequence_length", "64",
               "--batch_size", "8", "--acc_steps", "2", "--vocab_size", "512", "--dataset", "synthetic-zipf",
               "--datasets_dir", str(tmp_path / "data"), "--opt", "dana-star-mk4", "--kappa", "0.85", "--clipsnr", "2.0",
               "--wd_decaying", "--wd_ts", "5", "--lr", "1e-3", "--warmup_steps", "2", "--scheduler", "cos_inf",
               "--eval_interval", "4", "--eval_batches", "2", "--log_interval", "2", "--latest_ckpt_interval", "4",
               "--results_base_folder", str(tmp_path / "exps"), "--device", "cpu", "--dtype", "float32",
               "--distributed_backend", "fsdp", "--seed", "3", *extra]
        env = {**os.environ, "ADANA_FSDP_CPU": "1", "OMP_NUM_THREADS": "1"}
        p = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600, env=env)
        assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
        return p.stdout + p.stderr

    out = launch(["--iterations", "8", "--iterations_to_run", "5"])
    exp = _exp_dir(tmp_path / "exps")
    latest = exp / "ckpts" / "latest"
    # the reference's FSDP layout: a torch.distributed.checkpoint directory (index + one data file per rank)
    assert (latest / "sharded" / ".metadata").exists() and len(list((latest / "sharded").glob("*.distcp"))) == 2
    assert (latest / "meta.pt").exists() and (latest / "worker_1.pt").exists()
    assert torch.load(latest / "meta.pt", map_location="cpu", weights_only=False)["itr"] == 5
    out = launch(["--iterations", "8", "--auto_resume"])
    assert ">Eval: Iter=8" in out
    rows = [json.loads(l) for l in (exp / "metrics.jsonl").read_text().splitlines()]
    iters = [r["iter"] for r in rows if "train/loss" in r]
    assert iters == sorted(set(iters)) and iters[-1] == 8                     # no iteration logged twice
    assert json.loads((exp / "summary.json").read_text())["args"]["distributed_backend"] == "fsdp"
    # the sharded checkpoint can be read without an engine or a process group: inference loads it
    from adana_b200 import inference
    from adana_b200.train.checkpoint import full_state_from_sharded

    full = full_state_from_sharded(exp / "ckpts" / "latest" / "sharded")
    model = inference.load_model(exp)
    params = dict(model.named_parameters())
    assert set(full) == set(params)
    for k, v in full.items():
        assert v.shape == params[k].shape and torch.isfinite(v).all()
        assert torch.equal(v, params[k].detach().float())
    moments = full_state_from_sharded(exp / "ckpts" / "latest" / "sharded", "v")
    assert set(moments) == set(full) and all((t >= 0).all() for t in moments.values())
    toks = list(inference.generate_tokens(model, torch.tensor([[1, 2, 3]]), 4, temperature=0.0))
    assert len(toks) == 4 and all(t.shape == (1, 1) for t in toks)


@pytest.mark.timeout(600)
def test_two_rank_sharded_muon_cli_run(tmp_path):
    """`--opt d-muon` under the sharded engine: gather -> Newton-Schulz -> scatter through the command line."""
    import os
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1", "--nnodes=1", "--nproc-per-node", "2", "-m", "adana_b200.main", "--model", "qwen3", "--n_layer", "2", "--n_head", "2",
           "--n_embd", "64", "--qkv_dim", "32", "--mlp_hidden_dim", "128", "--sequence_length", "64", "--batch_size", "8",
           "--acc_steps", "2", "--vocab_size", "512", "--dataset", "synthetic-zipf", "--datasets_dir", str(tmp_path / "data"),
           "--opt", "d-muon", "--momentum", "0.95", "--nesterov", "True", "--beta1", "0.8", "--beta2", "0.999", "--lr", "2e-3",
           "--iterations", "12", "--warmup_steps", "2", "--scheduler", "cos_inf", "--eval_interval", "3", "--eval_batches", "2",
           "--log_interval", "2", "--results_base_folder", str(tmp_path / "exps"), "--device", "cpu", "--dtype", "float32",
           "--distributed_backend", "fsdp", "--seed", "3"]
    env = {**os.environ, "ADANA_FSDP_CPU": "1", "OMP_NUM_THREADS": "1"}
    p = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=500, env=env)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    rows = [json.loads(l) for l in (_exp_dir(tmp_path / "exps") / "metrics.jsonl").read_text().splitlines()]
    val = [r["val/loss"] for r in rows if "val/loss" in r] + [r["final-val/loss"] for r in rows if "final-val/loss" in r]
    # (the run is seeded: the same numbers every time; the loss of the last evaluation is below the untrained one)
    assert len(val) >= 4 and all(v == v for v in val) and val[-1] < val[0], val


@pytest.mark.timeout(900)
def test_four_rank_dp_by_tp_cli_run_saves_and_resumes(tmp_path):
    """`--tp_size 2` on four CPU ranks (2 data-parallel x 2 tensor-parallel) through the command line on the kernel engine:
    trains, writes one full checkpoint assembled over both groups, and a second run resumes from it."""
    import os

    base = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1", "--nnodes=1",
            "--nproc-per-node", "4", "-m", "adana_b200.main", "--model", "enoki", "--n_layer", "2", "--n_head", "4",
            "--n_embd", "64", "--qkv_dim", "16", "--mlp_hidden_dim", "128", "--sequence_length", "64", "--batch_size", "8",
            "--acc_steps", "2", "--vocab_size", "512", "--dataset", "synthetic-zipf", "--datasets_dir", str(tmp_path / "data"),
            "--opt", "dana-star-mk4", "--lr", "2e-3", "--warmup_steps", "2", "--scheduler", "cos_inf", "--eval_interval", "4",
            "--eval_batches", "2", "--log_interval", "2", "--results_base_folder", str(tmp_path / "exps"), "--device", "cpu",
            "--dtype", "float32", "--distributed_backend", "fsdp", "--tp_size", "2", "--seed", "3", "--permanent_ckpt_interval", "4"]
    env = {**os.environ, "ADANA_FSDP_CPU": "1", "OMP_NUM_THREADS": "1"}
    p = subprocess.run(base + ["--iterations", "8"], cwd=ROOT, capture_output=True, text=True, timeout=400, env=env)
    assert p.returncode == 0, "\n".join(l for l in p.stderr.splitlines() if "Error" in l or "error" in l)[-3000:]
    exp = _exp_dir(tmp_path / "exps")
    rows = [json.loads(l) for l in (exp / "metrics.jsonl").read_text().splitlines()]
    val = [r["val/loss"] for r in rows if "val/loss" in r] + [r["final-val/loss"] for r in rows if "final-val/loss" in r]
    assert len(val) >= 2 and all(v == v for v in val) and val[-1] < val[0], val
    ckpts = sorted((exp / "ckpts").glob("*/main.pt"))
    assert ckpts, list((exp / "ckpts").rglob("*"))
    sd = torch.load(ckpts[-1], map_location="cpu", weights_only=False)
    assert tuple(sd["model"]["transformer.h.0.attn.c_attn.weight"].shape) == (3 * 4 * 16, 64)      # full, not a tp part
    assert tuple(sd["model"]["transformer.h.0.mlp.c_proj.weight"].shape) == (64, 128)
    p = subprocess.run(base + ["--iterations", "10", "--resume_from", str(ckpts[-1].parent)], cwd=ROOT, capture_output=True,
                       text=True, timeout=400, env=env)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]


@pytest.mark.timeout(900)
def test_rank_that_leaves_ends_the_job_and_the_relaunch_resumes_from_the_last_checkpoint(tmp_path):
    """Job-level recovery, failure made on the host: rank 1 of a two-rank FSDP run leaves at iteration 6 (between
    steps).  The survivor must not hang: the launcher ends the job with a non-zero code, the checkpoint of iteration 4
    is complete, and a relaunch with --auto_resume — here on ONE rank, the elastic case — carries on from it."""
    import os

    def launch(nproc, extra, env_extra=None, expect_ok=True):
        cmd = [*torchrun(nproc), "-m", "adana_b200.main", "--model", "enoki", "--n_layer", "2",
               "--n_head", "2", "--n_embd", "64", "--qkv_dim", "32", "--mlp_hidden_dim", "128", "--sequence_length", "64",
               "--batch_size", "8", "--acc_steps", "2", "--vocab_size", "512", "--dataset", "synthetic-zipf",
               "--datasets_dir", str(tmp_path / "data"), "--opt", "dana-star-mk4", "--kappa", "0.85", "--clipsnr", "2.0",
               "--wd_decaying", "--wd_ts", "5", "--lr", "1e-3", "--warmup_steps", "2", "--scheduler", "cos_inf",
               "--eval_interval", "4", "--eval_batches", "2", "--log_interval", "1", "--latest_ckpt_interval", "4",
               "--results_base_folder", str(tmp_path / "exps"), "--device", "cpu", "--dtype", "float32",
               "--distributed_backend", "fsdp", "--seed", "3", "--heartbeat_timeout", "5", "--experiment_name", "recover", *extra]
        env = {**os.environ, "ADANA_FSDP_CPU": "1", "OMP_NUM_THREADS": "1", **(env_extra or {})}
        p = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600, env=env)
        assert (p.returncode == 0) == expect_ok, p.stdout[-2000:] + p.stderr[-2000:]
        return p.stdout + p.stderr

    t0 = time.time()
    out = launch(2, ["--iterations", "10"], {"ADANA_FAULT_EXIT": "1:6"}, expect_ok=False)
    assert time.time() - t0 < 300                                   # ended by the failure, not by the test's timeout
    assert "[Fault] leaving at iteration 6" in out and "Train: Iter=10" not in out
    exp = _exp_dir(tmp_path / "exps")
    latest = exp / "ckpts" / "latest"
    assert torch.load(latest / "meta.pt", map_location="cpu", weights_only=False)["itr"] == 4
    assert len(list((latest / "sharded").glob("*.distcp"))) == 2 and not (exp / "summary.json").exists()
    out = launch(1, ["--iterations", "10", "--auto_resume"])
    assert ">Eval: Iter=10" in out and (exp / "summary.json").exists()
    rows = [json.loads(l) for l in (exp / "metrics.jsonl").read_text().splitlines()]
    iters = [r["iter"] for r in rows if "train/loss" in r]
    assert iters[-1] == 10 and 5 in iters and all(r["train/loss"] == r["train/loss"] for r in rows if "train/loss" in r)


@pytest.mark.timeout(600)
def test_two_rank_moe_run_with_expert_parallel_layers(tmp_path):
    """Qwen3-Next with routed experts split over two data-parallel CPU ranks: training, the evaluations (every rank
    takes part: the expert exchange is collective) and the final summary go through."""
    import os

    cmd = [*torchrun(2), "-m", "adana_b200.main", "--model", "qwen3next", "--moe", "--moe_num_experts", "4",
           "--moe_num_experts_per_tok", "2", "--n_layer", "2", "--n_head", "2", "--n_embd", "64", "--qkv_dim", "32",
           "--mlp_hidden_dim", "128", "--sequence_length", "128", "--batch_size", "16", "--acc_steps", "2", "--vocab_size", "512",
           "--dataset", "synthetic-zipf", "--datasets_dir", str(tmp_path / "data"), "--opt", "adamw", "--lr", "1e-3",
           "--iterations", "6", "--warmup_steps", "2", "--eval_interval", "3", "--eval_batches", "2", "--log_interval", "1",
           "--latest_ckpt_interval", "0", "--grad_clip", "0.5", "--results_base_folder", str(tmp_path / "exps"),
           "--device", "cpu", "--dtype", "float32", "--distributed_backend", "gloo", "--seed", "2"]
    p = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=500, env={**os.environ, "OMP_NUM_THREADS": "1"})
    out = p.stdout + p.stderr
    assert p.returncode == 0, out[-3000:]
    assert ">Eval: Iter=3" in out and ">Eval: Iter=6" in out and "Train: Iter=6" in out
    rows = [json.loads(l) for l in (_exp_dir(tmp_path / "exps") / "metrics.jsonl").read_text().splitlines()]
    losses = [r["train/loss"] for r in rows if "train/loss" in r]
    assert len(losses) == 6 and all(l == l for l in losses)


@pytest.mark.timeout(900)
def test_two_rank_library_fsdp_model_saves_a_dcp_checkpoint_and_resumes(tmp_path):
    """A model the kernel engine does not take (Qwen3 with tied embeddings) runs under torch's FSDP2: its checkpoint is
    a torch.distributed.checkpoint directory plus meta.pt, as the reference writes under FSDP (src/optim/utils.py:
    275-298), not rank 0's DTensor shards in a main.pt; the relaunch resumes from it and inference reads it."""
    import os

    def launch(extra):
        cmd = [*torchrun(2), "-m", "adana_b200.main", "--model", "qwen3", "--weight_tying", "True", "--n_layer", "2",
               "--n_head", "2", "--n_embd", "64", "--qkv_dim", "32", "--mlp_hidden_dim", "128", "--sequence_length", "128",
               "--batch_size", "8", "--acc_steps", "2", "--vocab_size", "512", "--dataset", "synthetic-zipf",
               "--datasets_dir", str(tmp_path / "data"), "--opt", "adamw", "--lr", "1e-3", "--warmup_steps", "2",
               "--eval_interval", "100", "--eval_batches", "2", "--log_interval", "1", "--latest_ckpt_interval", "3",
               "--results_base_folder", str(tmp_path / "exps"), "--device", "cpu", "--dtype", "float32",
               "--distributed_backend", "fsdp", "--seed", "3", "--iterations", "6", *extra]
        p = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600,
                           env={**os.environ, "ADANA_FSDP_CPU": "1", "OMP_NUM_THREADS": "1"})
        assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
        return p.stdout + p.stderr

    launch(["--iterations_to_run", "3"])
    latest = _exp_dir(tmp_path / "exps") / "ckpts" / "latest"
    assert (latest / "sharded" / ".metadata").exists() and len(list((latest / "sharded").glob("*.distcp"))) == 2
    assert not (latest / "main.pt").exists()
    assert torch.load(latest / "meta.pt", map_location="cpu", weights_only=False)["itr"] == 3
    out = launch(["--auto_resume"])
    assert "Train: Iter=4" in out and "Train: Iter=6" in out and "Train: Iter=1 " not in out
    from adana_b200 import inference

    model = inference.load_model(_exp_dir(tmp_path / "exps"))
    assert all(torch.isfinite(p).all() for p in model.parameters())
    assert model.lm_head.weight is model.transformer.wte.weight
