"""Checkpoint I/O.

On-disk layouts (a run directory holds `ckpts/latest` and `ckpts/<iteration>`):

  replicated / single   `<ckpt>/main.pt` = {"model", "optimizer", "scheduler", "itr"} — the
                        reference's file (src/optim/utils.py:300-310), readable by both sides,
                        including the `_orig_mod.` / `module.` key prefixes of compiled / DDP runs.
  sharded (fsdp)        `<ckpt>/sharded/` = a `torch.distributed.checkpoint` directory holding
                        {"model", "optimizer"} keyed by parameter name, and `<ckpt>/meta.pt` =
                        {"scheduler", "itr"}: the reference's layout (src/optim/utils.py:275-298), which
                        its own `dcp.load` reads.  Every rank writes only the rectangles of each tensor
                        that its flat shards cover (train/dcp_format.py), no gather, so the time to
                        checkpoint does not grow with the model; loading with a different world size
                        reads the overlapping chunks.  meta.pt is written last: a directory that has it
                        is complete.  `export_full()` / `import_dcp()` convert to `main.pt` and from a
                        directory written by the reference.
  every rank            `<ckpt>/worker_{rank}.pt` = RNG states (torch CPU/GPU, numpy, python) and
                        the data-reader position (reference src/optim/utils.py:364-415).

Writes go to a temporary name and are renamed into place, so an interrupted job never leaves a
torn file; with `SLURM_TMPDIR` set, files are written node-locally and a background thread
rsyncs + atomically renames them into the project directory
(reference src/optim/utils.py:15-71, 236-257).  `AsyncWriter` moves serialisation off the
training thread (`--async_checkpoint`).
"""
from __future__ import annotations

import json
import os
import random
import shutil
import subprocess
import threading
from pathlib import Path
from typing import Dict, Optional

import numpy as np
import torch
import torch.distributed as dist

_rsync_thread: Optional[threading.Thread] = None
_PREFIXES = ("_orig_mod.", "module.")


# ---- helpers ------------------------------------------------------------------------------------------
def _rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def _atomic_save(obj, path: Path) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_name(path.name + f".tmp{os.getpid()}")
    torch.save(obj, tmp)
    os.replace(tmp, path)


def _load(path, map_location="cpu"):
    try:
        return torch.load(path, map_location=map_location)
    except Exception:
        return torch.load(path, map_location=map_location, weights_only=False)


def strip_prefixes(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in sd.items():
        changed = True
        while changed:
            changed = False
            for p in _PREFIXES:
                if k.startswith(p):
                    k, changed = k[len(p):], True
        out[k] = v
    return out


class AsyncWriter:
    """Serialises checkpoint payloads on a background thread (one write in flight at a time)."""

    def __init__(self):
        self._thread: Optional[threading.Thread] = None
        self.error: Optional[BaseException] = None

    def submit(self, obj, path: Path):
        self.wait()

        def run():
            try:
                _atomic_save(obj, path)
            except BaseException as e:  # surfaced on the next wait()
                self.error = e

        self._thread = threading.Thread(target=run, daemon=True, name="adana-ckpt-writer")
        self._thread.start()

    def wait(self):
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        if self.error is not None:
            e, self.error = self.error, None
            raise RuntimeError(f"asynchronous checkpoint write failed: {e}") from e


_async_writer = AsyncWriter()


# ---- node-local staging + rsync (SLURM) ------------------------------------------------------------------
def _local_dir(ckpt_dir: Path):
    tmp = os.environ.get("SLURM_TMPDIR")
    if tmp:
        return Path(tmp) / "ckpts" / ckpt_dir.name, ckpt_dir, True
    return ckpt_dir, ckpt_dir, False


def wait_for_rsync():
    global _rsync_thread
    if _rsync_thread is not None:
        _rsync_thread.join()
        _rsync_thread = None


def rsync_if_slurm(ckpt_dir: Path):
    """Rank 0, after all ranks finished writing: copy the node-local checkpoint to the project
    directory in the background and swap it into place with a rename."""
    global _rsync_thread
    local, project, is_slurm = _local_dir(ckpt_dir)
    if not is_slurm:
        return

    def run():
        staging = project.with_name(project.name + ".incoming")
        staging.mkdir(parents=True, exist_ok=True)
        try:
            subprocess.run(["rsync", "-a", "--delete", f"{local}/", f"{staging}/"], check=True)
        except (subprocess.CalledProcessError, OSError) as e:
            # a failed or partial copy must not replace the last good checkpoint (the reference keeps the old one
            # too: src/optim/utils.py:19-51)
            print(f"[Checkpoint] rsync of {local} failed ({e}); keeping the previous {project}")
            shutil.rmtree(staging, ignore_errors=True)
            return
        old = project.with_name(project.name + ".old")
        if project.exists():
            if old.exists():
                shutil.rmtree(old, ignore_errors=True)
            os.replace(project, old)
        os.replace(staging, project)
        shutil.rmtree(old, ignore_errors=True)

    wait_for_rsync()
    _rsync_thread = threading.Thread(target=run, daemon=True, name="adana-ckpt-rsync")
    _rsync_thread.start()


# ---- model / optimizer -------------------------------------------------------------------------------------
def _engine_of(model):
    return getattr(model, "_engine", None) or getattr(getattr(model, "module", None), "_engine", None)


def _is_sharded(model) -> bool:
    eng = _engine_of(model)
    return eng is not None and eng.sharded


def model_state_dict(model) -> Dict[str, torch.Tensor]:
    """Full fp32 state dict under every backend (collective when the engine is sharded)."""
    eng = _engine_of(model)
    if eng is not None and (eng.sharded or getattr(eng, "tp", None) is not None):
        return {k: v.cpu() for k, v in eng.full_param_dict("master").items()}
    if isinstance(model, torch.nn.parallel.DistributedDataParallel):
        model = model.module
    return model.state_dict()


def save_checkpoint(model, opt, scheduler, itr, ckpt_dir: Path, distributed_backend=None, async_write=False):
    ckpt_dir = Path(ckpt_dir)
    local, _, is_slurm = _local_dir(ckpt_dir)
    if is_slurm:
        wait_for_rsync()
    local.mkdir(parents=True, exist_ok=True)
    eng = _engine_of(model)
    sched_sd = scheduler.state_dict() if scheduler is not None else None
    if eng is not None and getattr(eng, "tp", None) is not None:
        # tensor parallelism: every rank takes part in reassembling the full tensors (over its data-parallel group and
        # over tp), global rank 0 writes one reference-format main.pt that any layout can load again
        ckpt = {"model": model_state_dict(model), "optimizer": _to_cpu(opt.state_dict()), "scheduler": sched_sd, "itr": itr}
        if _rank() == 0:
            _atomic_save(ckpt, local / "main.pt")
        return
    if eng is not None and eng.sharded:
        # `<ckpt>/sharded/` is a torch.distributed.checkpoint directory, as in the reference (src/optim/utils.py:
        # 275-298): every rank writes the rectangles of every tensor that its flat shards cover (train/dcp_format.py).
        # The call is collective and returns when all ranks' files and the index are on disk; only then does rank 0
        # write meta.pt, so a directory with a meta.pt is complete.
        from .dcp_format import save_engine_state

        _async_writer.wait()
        if eng.rank == 0:
            stale = local / "meta.pt"
            if stale.exists():
                stale.unlink()
        save_engine_state(eng, opt, local / "sharded")
        if eng.rank == 0:
            _atomic_save({"scheduler": sched_sd, "itr": itr}, local / "meta.pt")
        return
    if _is_torch_fsdp(model):
        # models without a kernel path run under torch's FSDP2: their parameters are DTensor shards, saved the way the
        # reference saves them (src/optim/utils.py:275-298) -- a collective torch.distributed.checkpoint write of the
        # state dictionaries, then meta.pt on rank 0
        import torch.distributed.checkpoint as dcp
        from torch.distributed.checkpoint.state_dict import get_model_state_dict, get_optimizer_state_dict

        if _rank() == 0 and (local / "meta.pt").exists():
            (local / "meta.pt").unlink()
        dcp.save({"model": get_model_state_dict(model), "optimizer": _fsdp_optimizer_state(model, opt)},
                 checkpoint_id=str(local / "sharded"))
        if _rank() == 0:
            _atomic_save({"scheduler": sched_sd, "itr": itr}, local / "meta.pt")
        return
    if _rank() != 0:
        return
    if any(getattr(p, "_adana_rank_local", False) for p in model.parameters()):
        print("[Checkpoint] WARNING: expert-parallel layers keep each rank's experts on that rank only; main.pt holds "
              "rank 0's.  Train with --no_expert_parallel when the run has to be resumed from its checkpoints.")
    ckpt = {"model": model_state_dict(model), "optimizer": opt.state_dict(), "scheduler": sched_sd, "itr": itr}
    if async_write:
        ckpt = {k: (_to_cpu(v)) for k, v in ckpt.items()}
        _async_writer.submit(ckpt, local / "main.pt")
    else:
        _atomic_save(ckpt, local / "main.pt")


def _is_torch_fsdp(model) -> bool:
    """True for a module that torch's `fully_shard` wrapped (its parameters are DTensors)."""
    try:
        from torch.distributed.tensor import DTensor
    except ImportError:
        return False
    return any(isinstance(p, DTensor) for p in model.parameters())


def _fsdp_optimizer_state(model, opt):
    """`get_optimizer_state_dict`, which takes one dry step (zero gradients, zero learning rate) when the optimizer has
    no state yet; a schedule-free optimizer that the trainer has put into evaluation mode for the checkpoint refuses
    steps, so it is switched to training mode around the call."""
    from torch.distributed.checkpoint.state_dict import get_optimizer_state_dict

    parked = bool(opt.param_groups) and opt.param_groups[0].get("train_mode") is False and hasattr(opt, "train")
    if parked:
        opt.train()
    try:
        return get_optimizer_state_dict(model, opt)
    finally:
        if parked:
            opt.eval()


def _to_cpu(obj):
    if torch.is_tensor(obj):
        return obj.detach().cpu().clone()
    if isinstance(obj, dict):
        return {k: _to_cpu(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_cpu(v) for v in obj)
    return obj


def _load_sharded(eng, opt, sharded_dir: Path):
    layout = json.loads((sharded_dir / "layout.json").read_text())
    saved_world = layout["world"]
    files = {}
    by_name = {u["name"]: u for u in layout["units"]}
    opt_step = None
    # A directory whose rank files come from different saves (a crash between two ranks' writes, a partial copy) must
    # not be resumed from: every rank file carries the iteration it was written at.
    meta_path = sharded_dir.parent / "meta.pt"
    want_itr = _load(meta_path).get("itr") if meta_path.exists() else None
    for r in range(saved_world):
        if not (sharded_dir / f"rank{r:05d}.pt").exists():
            raise RuntimeError(f"sharded checkpoint {sharded_dir} is incomplete: rank{r:05d}.pt is missing")

    def saved(rank):      # (each rank opens only the files that overlap its shard; together the ranks open all)
        if rank not in files:
            files[rank] = _load(sharded_dir / f"rank{rank:05d}.pt")
            got = files[rank].get("itr")
            if want_itr is not None and got is not None and int(got) != int(want_itr):
                raise RuntimeError(f"sharded checkpoint {sharded_dir} is inconsistent: rank{rank:05d}.pt was written at "
                                   f"iteration {got}, meta.pt at {want_itr}")
        return files[rank]

    for u in eng.units:
        lu = by_name[u.layout.name]
        if [s["name"] for s in lu["slots"]] != [s.name for s in u.layout.slots]:
            raise RuntimeError(f"checkpoint layout of {u.layout.name} does not match this model")
        s_shard = lu["padded"] // saved_world
        lo, hi = u.shard_off, u.shard_off + u.shard_len
        hi_used = min(hi, lu["numel"])
        keys = None
        for r in range(saved_world):
            a, b = max(lo, r * s_shard), min(hi_used, (r + 1) * s_shard)
            if a >= b:
                continue
            entry = saved(r)["units"][u.layout.name]
            opt_step = saved(r).get("opt_step", opt_step)
            keys = [k for k in entry if k != "master"]
            u.ensure_state(keys)
            for k, t in entry.items():
                dst = u.master if k == "master" else u.state[k]
                dst[a - lo:b - lo].copy_(t[a - r * s_shard:b - r * s_shard])
    if opt is not None and opt_step is not None and hasattr(opt, "step_count"):
        opt.step_count = int(opt_step)
    if opt is not None and hasattr(opt, "inner"):
        own = saved(eng.rank) if saved_world == eng.world else None
        if own is None or "per_tensor_opt" not in own:
            raise RuntimeError("the state of a per-tensor optimizer under the sharded engine can only be restored on the "
                               f"world size it was saved with ({saved_world}); this run has {eng.world} ranks")
        opt.load_state_dict(own["per_tensor_opt"])
        eng.refresh_from_master()
        return
    any_file = saved(0)
    if opt is not None and "param_groups" in any_file:
        for g, sg in zip(opt.param_groups, any_file["param_groups"]):
            for k, v in sg.items():
                g[k] = v
    eng.refresh_from_master()


def full_state_from_sharded(sharded_dir: Path, which: str = "master") -> Dict[str, torch.Tensor]:
    """Reassemble the full fp32 tensors (`which`: master | m | v | tau) of a sharded checkpoint without an engine or a
    process group: name -> tensor, from `layout.json` and the `rank*.pt` files of any world size.  What inference
    and single-file export need from an FSDP run (the reference's inference reads DDP/single checkpoints only,
    inference.py:165-191)."""
    sharded_dir = Path(sharded_dir)
    if (sharded_dir / ".metadata").exists():
        model_sd, opt_sd = import_dcp(sharded_dir)
        if which == "master":
            return model_sd
        names = {"m": ("m", "exp_avg", "exp_avg_fast"), "v": ("v", "exp_avg_sq"), "tau": ("tau", "exp_avg_slow")}[which]
        out = {}
        for n, st in ((opt_sd or {}).get("state", {}) or {}).items():
            for k in names:
                if isinstance(st, dict) and k in st:
                    out[n] = st[k]
        return out
    layout = json.loads((sharded_dir / "layout.json").read_text())
    world = layout["world"]
    files = [_load(sharded_dir / f"rank{r:05d}.pt") for r in range(world)]
    out: Dict[str, torch.Tensor] = {}
    for lu in layout["units"]:
        parts = []
        for r in range(world):
            entry = files[r]["units"][lu["name"]]
            if which not in entry:
                parts = None
                break
            parts.append(entry[which].reshape(-1).float())
        if parts is None:
            continue
        flat = torch.cat(parts)[:lu["numel"]]
        for sl in lu["slots"]:
            n = 1
            for d in sl["shape"]:
                n *= d
            out[sl["name"]] = flat[sl["offset"]:sl["offset"] + n].view(sl["shape"]).clone()
    return out


def load_checkpoint(model, opt, scheduler, ckpt_path, device="cpu", distributed_backend=None) -> int:
    """Restores model, optimizer and scheduler; returns the iteration stored in the checkpoint."""
    ckpt_path = Path(ckpt_path)
    ckpt_dir = ckpt_path.parent if ckpt_path.suffix == ".pt" else ckpt_path
    eng = _engine_of(model)
    if (ckpt_dir / "sharded" / ".metadata").exists() and eng is not None and eng.sharded:
        from .dcp_format import load_engine_state

        if not (ckpt_dir / "meta.pt").exists():
            raise RuntimeError(f"sharded checkpoint {ckpt_dir} is incomplete: meta.pt (written last) is missing")
        load_engine_state(eng, opt, ckpt_dir / "sharded")
        meta = _load(ckpt_dir / "meta.pt")
        if scheduler is not None and meta.get("scheduler") is not None:
            scheduler.load_state_dict(meta["scheduler"])
        return meta["itr"]
    if (ckpt_dir / "sharded" / "layout.json").exists() and eng is not None:
        _load_sharded(eng, opt, ckpt_dir / "sharded")      # the flat-shard files earlier versions wrote
        meta = _load(ckpt_dir / "meta.pt")
        if scheduler is not None and meta.get("scheduler") is not None:
            scheduler.load_state_dict(meta["scheduler"])
        return meta["itr"]
    if _is_torch_fsdp(model) and (ckpt_dir / "sharded" / ".metadata").exists():
        # the reference's loader (src/optim/utils.py:328-337): read into the sharded state dictionaries, hand them back
        import torch.distributed.checkpoint as dcp
        from torch.distributed.checkpoint.state_dict import (get_model_state_dict, get_optimizer_state_dict,
                                                             set_model_state_dict, set_optimizer_state_dict)

        if not (ckpt_dir / "meta.pt").exists():
            raise RuntimeError(f"sharded checkpoint {ckpt_dir} is incomplete: meta.pt (written last) is missing")
        state = {"model": get_model_state_dict(model), "optimizer": _fsdp_optimizer_state(model, opt)}
        # (the dry step that fills an empty optimizer state can create entries a trained state no longer carries,
        # e.g. a pending copy of the last gradient: entries absent from the checkpoint keep their fresh value)
        from torch.distributed.checkpoint.default_planner import DefaultLoadPlanner

        dcp.load(state, checkpoint_id=str(ckpt_dir / "sharded"), planner=DefaultLoadPlanner(allow_partial_load=True))
        set_model_state_dict(model, state["model"])
        set_optimizer_state_dict(model, opt, state["optimizer"])
        meta = _load(ckpt_dir / "meta.pt")
        if scheduler is not None and meta.get("scheduler") is not None:
            scheduler.load_state_dict(meta["scheduler"])
        return meta["itr"]
    if (ckpt_dir / "sharded").is_dir() and not (ckpt_dir / "main.pt").exists():
        model_sd, opt_sd = import_dcp(ckpt_dir / "sharded")
        meta = _load(ckpt_dir / "meta.pt")
        ckpt = {"model": model_sd, "optimizer": opt_sd, "scheduler": meta.get("scheduler"), "itr": meta["itr"]}
    else:
        ckpt = _load(ckpt_dir / "main.pt")
    sd = strip_prefixes(ckpt["model"])
    if eng is not None:
        eng.load_full_param_dict({k: v.to(eng.device) for k, v in sd.items()})
    else:
        target = model.module if isinstance(model, torch.nn.parallel.DistributedDataParallel) else model
        target.load_state_dict(sd)
    if opt is not None and ckpt.get("optimizer") is not None:
        opt.load_state_dict(ckpt["optimizer"])
    if scheduler is not None and ckpt.get("scheduler") is not None:
        scheduler.load_state_dict(ckpt["scheduler"])
    return ckpt["itr"]


def export_full(model, opt, scheduler, itr, out_path: Path):
    """Gather a sharded run into a single reference-format `main.pt` (all ranks call; rank 0 writes)."""
    sd = model_state_dict(model)
    osd = opt.state_dict()
    if _rank() == 0:
        _atomic_save({"model": sd, "optimizer": _to_cpu(osd),
                      "scheduler": scheduler.state_dict() if scheduler is not None else None, "itr": itr},
                     Path(out_path))


def import_dcp(sharded_dir: Path):
    """Read a `torch.distributed.checkpoint` directory (as written by the reference under FSDP)
    into plain full tensors: returns (model_state_dict, optimizer_state_dict | None)."""
    from torch.distributed.checkpoint import FileSystemReader
    from torch.distributed.checkpoint.state_dict_loader import _load_state_dict
    from torch.distributed.checkpoint.default_planner import _EmptyStateDictLoadPlanner

    sd: Dict = {}
    _load_state_dict(sd, storage_reader=FileSystemReader(str(sharded_dir)),
                     planner=_EmptyStateDictLoadPlanner(), no_dist=True)
    return strip_prefixes(sd.get("model", {})), sd.get("optimizer")


# ---- per-rank worker state -------------------------------------------------------------------------------------
def save_worker_state(ckpt_dir: Path, train_reader=None, verbose=True):
    local, _, _ = _local_dir(Path(ckpt_dir))
    state = {"rng_torch_cpu": torch.random.get_rng_state(), "rng_np": np.random.get_state(),
             "rng_python": random.getstate(), "rng_torch_gpu": None}
    if torch.cuda.is_available():
        try:
            state["rng_torch_gpu"] = torch.cuda.get_rng_state()
        except RuntimeError:
            pass
    rank = _rank()
    if train_reader is not None and hasattr(train_reader, "state_dict"):
        ds = train_reader.state_dict()
        state["dataloader_state"] = ds
        if verbose:
            inner = getattr(train_reader, "current_reader", train_reader)
            preview = inner.preview_next_samples(3) if hasattr(inner, "preview_next_samples") else None
            print(f"[Rank {rank}] Checkpoint: data_seed={getattr(train_reader, 'seed', None)}, "
                  f"file_idx={ds.get('current_file_idx')}, step={ds.get('step')}, next={preview}")
    _atomic_save(state, local / f"worker_{rank}.pt")


def load_worker_state(ckpt_dir: Path, train_reader=None, verbose=True):
    rank = _rank()
    path = Path(ckpt_dir) / f"worker_{rank}.pt"
    if not path.exists():
        print(f"[Rank {rank}] Warning: no worker state at {path}; RNG and data position start fresh")
        return
    state = _load(path)
    torch.random.set_rng_state(state["rng_torch_cpu"])
    if state.get("rng_torch_gpu") is not None and torch.cuda.is_available():
        try:
            torch.cuda.set_rng_state(state["rng_torch_gpu"])
        except RuntimeError:
            pass
    np.random.set_state(state["rng_np"])
    random.setstate(state["rng_python"])
    if train_reader is not None and "dataloader_state" in state:
        train_reader.load_state_dict(state["dataloader_state"])
        if verbose:
            inner = getattr(train_reader, "current_reader", train_reader)
            preview = inner.preview_next_samples(3) if hasattr(inner, "preview_next_samples") else None
            print(f"[Rank {rank}] Restored: data_seed={getattr(train_reader, 'seed', None)}, "
                  f"step={state['dataloader_state'].get('step')}, next={preview}")


def checkpoint_exists(ckpt_dir: Path) -> bool:
    ckpt_dir = Path(ckpt_dir)
    return (ckpt_dir / "main.pt").exists() or (ckpt_dir / "meta.pt").exists()


def finish_pending_shard_writes():
    """Blocks until this rank's asynchronous checkpoint file is on disk (re-raises a failed write)."""
    _async_writer.wait()


def finish_pending_writes():
    _async_writer.wait()
    wait_for_rsync()
