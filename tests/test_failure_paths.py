"""Failure paths that must stop a run instead of corrupting it: a device wait that timed out (status word),
a sharded checkpoint whose rank files come from different saves, a failed rsync of a checkpoint."""
import json
import subprocess
from pathlib import Path

import pytest
import torch

from adana_b200 import main as M
from adana_b200.train import checkpoint as ck
from adana_b200.train import loop as L


def _argv(tmp_path, extra=()):
    return ["--model", "enoki", "--n_layer", "2", "--n_head", "2", "--n_embd", "64", "--qkv_dim", "32", "--mlp_hidden_dim",
            "128", "--sequence_length", "32", "--batch_size", "4", "--vocab_size", "512", "--dataset", "synthetic-zipf",
            "--datasets_dir", str(tmp_path / "data"), "--opt", "dana-star-mk4", "--lr", "1e-3", "--iterations", "8",
            "--warmup_steps", "2", "--scheduler", "cos_inf", "--eval_interval", "100", "--eval_batches", "1",
            "--log_interval", "2", "--latest_ckpt_interval", "4", "--results_base_folder", str(tmp_path / "exps"),
            "--device", "cpu", "--dtype", "float32", "--distributed_backend", "single", *extra]


def test_timed_out_device_wait_stops_the_run_before_the_next_checkpoint(tmp_path, monkeypatch):
    """The status word is read on logging iterations and before every checkpoint; once it reports a timed-out wait
    the run raises, and the state computed after the timeout is never written."""
    seen = []

    def fake_status(self):
        seen.append(self.curr_iter)
        if self.curr_iter >= 3:          # "a peer flag wait ran out during iteration 3"
            raise RuntimeError("adana_b200 kernel reported: timeout: wait on a peer flag")

    monkeypatch.setattr(L.Trainer, "_read_device_status", fake_status)
    args, parser = M.get_args(_argv(tmp_path))
    with pytest.raises(RuntimeError, match="peer flag.*stops before this state is checkpointed"):
        M.main(args, parser)
    assert seen[0] == 0 and 2 in seen              # checked before the checkpoint at 0 and on the logging iteration 2
    exp = next((tmp_path / "exps").iterdir())
    saved = torch.load(exp / "ckpts" / "latest" / "main.pt", weights_only=False)
    assert saved["itr"] == 0                       # the checkpoint due at iteration 4 was not written


def test_incomplete_sharded_checkpoint_is_refused(tmp_path):
    """meta.pt is written last, after the collective write of the `torch.distributed.checkpoint` directory has
    returned on every rank: a directory without it (a crash during the write) is not resumed from, and a directory
    that lost a data file fails loudly instead of resuming with missing state."""
    from conftest import tiny_args
    from adana_b200.models.utils import get_model
    from adana_b200.runtime.engine import EngineOptimizer, attach

    a = tiny_args("enoki", opt="adamw")
    m = get_model(a)
    eng = attach(m, a, device="cpu")
    eng.sharded = True                     # one rank writing the sharded layout
    specs = m.get_parameter_group_specs()
    for g in specs:
        g["param_names"] = g["params"]
    opt = EngineOptimizer(eng, "adamw", a, specs)
    d = tmp_path / "latest"
    ck.save_checkpoint(m, opt, None, 7, d)
    assert (d / "sharded" / ".metadata").exists()
    assert ck.load_checkpoint(m, opt, None, d) == 7
    meta = (d / "meta.pt").read_bytes()
    (d / "meta.pt").unlink()
    with pytest.raises(RuntimeError, match="incomplete.*meta.pt"):
        ck.load_checkpoint(m, opt, None, d)
    (d / "meta.pt").write_bytes(meta)
    for f in (d / "sharded").glob("*.distcp"):
        f.unlink()
    with pytest.raises(BaseException, match="distcp|CheckpointException"):      # (torch's CheckpointException is a BaseException)
        ck.load_checkpoint(m, opt, None, d)


def test_failed_rsync_keeps_the_last_good_checkpoint(tmp_path, monkeypatch):
    project = tmp_path / "project" / "latest"
    project.mkdir(parents=True)
    (project / "main.pt").write_text("good")
    local = tmp_path / "node" / "ckpts" / "latest"
    local.mkdir(parents=True)
    (local / "main.pt").write_text("new")
    monkeypatch.setenv("SLURM_TMPDIR", str(tmp_path / "node"))

    def failing(cmd, check=False, **kw):
        assert check is True
        raise subprocess.CalledProcessError(23, cmd)

    monkeypatch.setattr(ck.subprocess, "run", failing)
    ck.rsync_if_slurm(project)
    ck.wait_for_rsync()
    assert (project / "main.pt").read_text() == "good" and not project.with_name("latest.incoming").exists()


def test_truncated_checkpoint_shard_fails_loudly(tmp_path):
    """A data file cut short (a disk that filled up, a copy that stopped) must not load as if it were complete."""
    from conftest import tiny_args
    from adana_b200.models.utils import get_model
    from adana_b200.runtime.engine import EngineOptimizer, attach

    a = tiny_args("enoki", opt="adamw")
    m = get_model(a)
    eng = attach(m, a, device="cpu")
    eng.sharded = True
    specs = m.get_parameter_group_specs()
    for g in specs:
        g["param_names"] = g["params"]
    opt = EngineOptimizer(eng, "adamw", a, specs)
    d = tmp_path / "latest"
    ck.save_checkpoint(m, opt, None, 3, d)
    before = {k: v.clone() for k, v in eng.full_param_dict("master").items()}
    f = next((d / "sharded").glob("*.distcp"))
    data = f.read_bytes()
    f.write_bytes(data[: len(data) // 2])
    with pytest.raises(BaseException):                       # torch's CheckpointException is a BaseException
        ck.load_checkpoint(m, opt, None, d)
    f.write_bytes(data)                                      # the intact file loads, and into the same numbers
    assert ck.load_checkpoint(m, opt, None, d) == 3
    for k, v in eng.full_param_dict("master").items():
        assert torch.equal(v, before[k])


def _stall_worker(rank, world, port, stall_rank, q):
    """Three ranks beat; one of them stops itself with SIGSTOP between steps (alive, but silent: its heartbeat thread
    stops with it).  The others must name it within the timeout."""
    import os
    import signal
    import time

    import torch.distributed as dist

    from adana_b200.runtime.watchdog import HeartbeatWatchdog, PeerFailure

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    wd = HeartbeatWatchdog.from_env(timeout_s=1.5)
    wd.beat(0)
    dist.barrier()
    wd.start()
    t0 = time.time()
    for it in range(1, 300):
        if rank == stall_rank and it == 3:
            q.put((rank, f"stopping pid {os.getpid()}"))
            time.sleep(0.5)                                  # the queue's feeder thread has to get the message out first
            os.kill(os.getpid(), signal.SIGSTOP)             # resumes only if the parent sends SIGCONT; it kills instead
        wd.beat(it)
        try:
            wd.raise_if_failed()
        except PeerFailure as e:
            wd.stop()
            q.put((rank, f"detected after {time.time() - t0:.1f}s: {e}"))
            q.close()
            q.join_thread()
            os._exit(0)                                      # no collective teardown with a stopped peer
        time.sleep(0.1)
    q.put((rank, "never detected"))
    q.close()
    q.join_thread()
    os._exit(0)


def test_watchdog_names_a_rank_that_is_alive_but_stopped():
    import socket
    import time

    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_stall_worker, args=(r, 3, port, 1, q)) for r in range(3)]
    for p in procs:
        p.start()
    got, deadline = {}, time.time() + 120
    try:
        while len(got) < 3 and time.time() < deadline:
            try:
                r, msg = q.get(timeout=1.0)
                got[r] = msg
            except Exception:
                pass
    finally:
        procs[1].kill()                                      # the stopped rank, by its own handle
        for p in procs:
            p.join(timeout=20)
            if p.is_alive():
                p.kill()
    assert got.get(1, "").startswith("stopping"), got
    for r in (0, 2):
        assert got.get(r, "").startswith("detected") and "rank 1" in got[r], got
