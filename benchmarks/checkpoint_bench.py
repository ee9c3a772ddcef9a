#!/usr/bin/env python
"""Sharded-checkpoint I/O against the disk: how long a save and a load of the sharded engine's state take, in bytes per
second, next to a plain sequential write and read of the same number of bytes by the same ranks.

    python benchmarks/checkpoint_bench.py [--ranks 2] [--heads 8] [--layers 6] [--repeats 3] [--dir /some/disk] [--json OUT]

Every rank is a CPU process (`gloo`); the engine keeps four fp32 vectors per parameter (master weights, m, v, tau), so
a model with P parameters writes about 16 P bytes over all ranks.  Timed, max over ranks and median over repeats:
  save     `train/checkpoint.py::save_checkpoint` (collective; returns when every rank's file and the index are on disk)
  load     `load_checkpoint` into a fresh engine of the same layout
  raw      each rank writes / reads its share of the same bytes with one `write` / `readinto` and an `fsync`
The ratio save / raw is what the checkpoint format costs on top of the disk (the layout bookkeeping, one copy into the
writer's buffers); nothing here needs a GPU: the engine's state lives in host memory at save time either way.
"""
import argparse
import json
import os
import statistics
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def _dir_bytes(p: Path) -> int:
    return sum(f.stat().st_size for f in p.rglob("*") if f.is_file())


def _worker(rank, world, port, a, out_q):
    import torch
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from adana_b200.config import flags
    from adana_b200.models.utils import get_model
    from adana_b200.parallel.comm import Comm
    from adana_b200.runtime.engine import EngineOptimizer, attach
    from adana_b200.train import checkpoint as ck

    def build():
        c = flags.defaults()
        c.model, c.n_head, c.n_layer, c.n_embd, c.qkv_dim = "enoki", a.heads, a.layers, 64 * a.heads, 64
        c.mlp_hidden_dim, c.sequence_length, c.vocab_size = 4 * 64 * a.heads, 64, 50304
        c.dtype, c.device, c.weight_tying, c.init_scheme, c.bias, c.dropout = "float32", "cpu", False, "ScaledGPT", False, 0.0
        c.opt, c.kappa, c.clipsnr, c.lr, c.weight_decay, c.wd_decaying, c.wd_ts = "dana-star-mk4", 0.85, 2.0, 1e-3, 0.1, True, 10.0
        c.acc_steps, c.grad_clip, c.z_loss_coeff = 1, 0.5, 0.0
        torch.manual_seed(0)
        m = get_model(c)
        eng = attach(m, c, comm=Comm(), sharded=True, device="cpu")
        specs = m.get_parameter_group_specs()
        for g in specs:
            g["param_names"] = g["params"]
        return m, eng, EngineOptimizer(eng, c.opt, c, specs), c

    m, eng, opt, c = build()
    x = torch.randint(0, c.vocab_size, (1, c.sequence_length))
    m.train()
    m(x, targets=x.roll(-1, 1))["loss"].backward()      # one step, so that every state vector holds numbers
    eng.grad_norm_and_clip(0.5)
    opt.step()
    opt.zero_grad()
    n_params = sum(s.numel for u in eng.units for s in u.layout.slots) if hasattr(eng.units[0].layout.slots[0], "numel") else \
        sum(p.numel() for p in m.parameters())
    base = Path(a.dir)
    saves, loads, raw_w, raw_r, size = [], [], [], [], 0

    def timed(fn):
        dist.barrier()
        t0 = time.perf_counter()
        fn()
        dist.barrier()
        t = torch.tensor([time.perf_counter() - t0], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    for rep in range(a.repeats):
        d = base / f"ckpt_{rep}"
        if a.profile and rank == 0 and rep == a.repeats - 1:
            import cProfile
            import pstats

            prof = cProfile.Profile()
            saves.append(timed(lambda: prof.runcall(ck.save_checkpoint, m, opt, None, 1, d)))
            pstats.Stats(prof).sort_stats("cumulative").print_stats(a.profile)
        else:
            saves.append(timed(lambda: ck.save_checkpoint(m, opt, None, 1, d)))
        if rank == 0:
            os.sync()
        dist.barrier()
        size = _dir_bytes(d)
        m2, eng2, opt2, _ = build()
        loads.append(timed(lambda: ck.load_checkpoint(m2, opt2, None, d / "main.pt")))
        share = size // world
        buf = bytearray(os.urandom(1 << 20) * (share >> 20)) if share >= (1 << 20) else bytearray(share)
        f = base / f"raw_{rep}_{rank}.bin"

        def write():
            with open(f, "wb") as fh:
                fh.write(buf)
                fh.flush()
                os.fsync(fh.fileno())

        def read():
            with open(f, "rb") as fh:
                fh.readinto(buf)

        raw_w.append(timed(write))
        raw_r.append(timed(read))
    if rank == 0:
        med = statistics.median
        out_q.put({"ranks": world, "parameters": int(n_params), "checkpoint_bytes": int(size),
                   "save_s": med(saves), "load_s": med(loads), "raw_write_s": med(raw_w), "raw_read_s": med(raw_r),
                   "save_MBps": size / med(saves) / 1e6, "load_MBps": size / med(loads) / 1e6,
                   "raw_write_MBps": (size // world) * world / med(raw_w) / 1e6, "raw_read_MBps": (size // world) * world / med(raw_r) / 1e6,
                   "save_over_raw_write": med(saves) / med(raw_w), "all_saves_s": saves, "all_loads_s": loads})
    dist.destroy_process_group()


def main():
    import socket

    import torch.multiprocessing as mp

    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=2)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--layers", type=int, default=6)
    ap.add_argument("--repeats", type=int, default=3)
    ap.add_argument("--dir", default=None)
    ap.add_argument("--json", default=None)
    ap.add_argument("--profile", type=int, default=0, help="print this many lines of rank 0's profile of the last save")
    a = ap.parse_args()
    with tempfile.TemporaryDirectory(dir=a.dir) as tmp:
        a.dir = tmp
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        procs = [ctx.Process(target=_worker, args=(r, a.ranks, port, a, q)) for r in range(a.ranks)]
        for p in procs:
            p.start()
        res = q.get(timeout=3600)
        for p in procs:
            p.join()
    print(json.dumps(res))
    if a.json:
        Path(a.json).write_text(json.dumps(res, indent=1))


if __name__ == "__main__":
    main()
