"""Sharded checkpoints in the `torch.distributed.checkpoint` directory layout.

The reference's FSDP runs save `dcp.save({"model": ..., "optimizer": ...}, "<ckpt>/sharded")` with state dicts
keyed by parameter name (src/optim/utils.py:275-289) and load them back into DTensor state dicts (328-337).  The
engine's state is not a set of DTensors: every rank holds one flat fp32 range per unit.  A range cuts a
parameter in up to three rectangles (the tail of a row, whole rows, the head of a row), and the DCP format
accepts any tiling of a tensor by rectangular chunks, so each rank writes exactly the rectangles it holds and
the directory that results is one the reference's `dcp.load` can read into its own sharding (and ours into any
world size: the reader intersects saved and wanted chunks).

`FlatPieces` is the object the DCP planners see instead of a tensor: it states its chunks
(`__create_write_items__` / `__create_chunk_list__`, the hooks DTensor uses) and hands out the views.
`save_engine_state` / `load_engine_state` build the `{"model", "optimizer"}` dictionaries around it.
"""
from __future__ import annotations

from pathlib import Path
from typing import Dict, List, Tuple

import torch


def _rectangles(a: int, b: int, shape: Tuple[int, ...]) -> List[Tuple[Tuple[int, ...], Tuple[int, ...], int, int]]:
    """Rectangles (offsets, sizes, flat begin, flat end) tiling the flat range [a, b) of a tensor of `shape`."""
    if a >= b:
        return []
    if len(shape) <= 1:
        return [((a,), (b - a,), a, b)]
    rows, cols = shape[0], 1
    for d in shape[1:]:
        cols *= d
    if len(shape) > 2:
        raise ValueError("flat ranges of tensors with more than two dimensions are not supported")
    out = []
    r0, c0 = divmod(a, cols)
    r1, c1 = divmod(b, cols)          # exclusive end: row r1, column c1
    if r0 == r1:                      # inside one row
        return [((r0, c0), (1, b - a), a, b)]
    pos = a
    if c0 != 0:                       # tail of the first row
        out.append(((r0, c0), (1, cols - c0), a, (r0 + 1) * cols))
        pos = (r0 + 1) * cols
        r0 += 1
    if r1 > r0:                       # whole rows
        out.append(((r0, 0), (r1 - r0, cols), pos, r1 * cols))
    if c1 != 0:                       # head of the last row
        out.append(((r1, 0), (1, c1), r1 * cols, b))
    return out


class FlatPieces:
    """What this rank holds of one parameter-shaped tensor: rectangles backed by views of the engine's flat shards."""

    def __init__(self, shape, dtype=torch.float32):
        self.shape = tuple(int(d) for d in shape)
        self.dtype = dtype
        self.chunks: List[Tuple[Tuple[int, ...], Tuple[int, ...], torch.Tensor]] = []

    def add_range(self, flat_view: torch.Tensor, a: int, b: int):
        """`flat_view` holds the elements [a, b) of the flattened tensor."""
        for offsets, sizes, x, y in _rectangles(a, b, self.shape):
            self.chunks.append((offsets, sizes, flat_view[x - a:y - a].view(sizes)))
        return self

    # ---- the hooks of torch.distributed.checkpoint's planners (DTensor implements the same three) ----------------
    def __create_chunk_list__(self):
        from torch.distributed.checkpoint.metadata import ChunkStorageMetadata

        return [ChunkStorageMetadata(offsets=torch.Size(o), sizes=torch.Size(s)) for o, s, _ in self.chunks]

    def __create_write_items__(self, fqn: str, obj):
        from torch.distributed.checkpoint.metadata import ChunkStorageMetadata, MetadataIndex, TensorProperties
        from torch.distributed.checkpoint.planner import TensorWriteData, WriteItem, WriteItemType

        items = []
        for o, s, t in self.chunks:
            items.append(WriteItem(
                index=MetadataIndex(fqn, torch.Size(o)), type=WriteItemType.SHARD,
                tensor_data=TensorWriteData(chunk=ChunkStorageMetadata(offsets=torch.Size(o), sizes=torch.Size(s)),
                                            properties=TensorProperties.create_from_tensor(t),
                                            size=torch.Size(self.shape))))
        return items

    def __get_tensor_shard__(self, index):
        want = tuple(index.offset) if index.offset is not None else None
        for o, _, t in self.chunks:
            if want is None or tuple(o) == want:
                return t
        raise ValueError(f"no chunk at offset {want} of {index.fqn}")


def _planners():
    from torch.distributed.checkpoint.default_planner import DefaultLoadPlanner, DefaultSavePlanner

    class SavePlanner(DefaultSavePlanner):
        def lookup_object(self, index):
            obj = self.state_dict.get(index.fqn)
            if isinstance(obj, FlatPieces):
                return obj.__get_tensor_shard__(index)
            return super().lookup_object(index)

    class LoadPlanner(DefaultLoadPlanner):
        def set_up_planner(self, state_dict, metadata=None, is_coordinator=False):
            # (the default set-up first rewrites every value it does not know to None)
            from torch.distributed.checkpoint._nested_dict import flatten_state_dict

            self.original_state_dict = state_dict
            self.state_dict, self.mappings = flatten_state_dict(state_dict)
            self.metadata = metadata
            self.is_coordinator = is_coordinator

        def lookup_tensor(self, index):
            obj = self.state_dict.get(index.fqn)
            if isinstance(obj, FlatPieces):
                return obj.__get_tensor_shard__(index)
            return super().lookup_tensor(index)

    return SavePlanner, LoadPlanner


# ---- engine <-> state dictionaries -------------------------------------------------------------------------------
def _pieces_of(eng, which: str) -> Dict[str, FlatPieces]:
    """name -> FlatPieces over this rank's part of `which` (master | m | v | tau) of every parameter."""
    out = {}
    for u in eng.units:
        src = u.master if which == "master" else u.state.get(which)
        lo, hi = u.shard_off, u.shard_off + u.shard_len
        for s in u.layout.slots:
            fp = FlatPieces(s.shape)
            a, b = max(s.offset, lo), min(s.offset + s.numel, hi)
            if src is not None and a < b:
                fp.add_range(src[a - lo:b - lo], a - s.offset, b - s.offset)
            out[s.name] = fp
    return out


def _state_keys(opt) -> Dict[str, str]:
    """engine moment name -> key in the per-parameter optimizer state (the per-tensor classes' names)."""
    from ..ops import optim as O
    from ..runtime.engine import FUSED_OPTS

    kind = FUSED_OPTS[opt.opt_name][0]
    if kind in (O.KIND_ADAMW, O.KIND_ADAMW_IWD):
        return {"m": "exp_avg", "v": "exp_avg_sq"}
    if kind in (O.KIND_ADEMAMIX, O.KIND_ADEMAMIX_IWD):
        return {"m": "exp_avg_fast", "v": "exp_avg_sq", "tau": "exp_avg_slow"}
    if kind == O.KIND_DANA_STAR:
        return {"m": "m", "v": "v", "tau": "tau"}
    return {"m": "m", "v": "v"}


_LOGGED_SCALARS = ("current_alpha", "gradient_norm", "auto_factor_mean", "current_kappa_factor", "m_norm")


def engine_state_dict(eng, opt, for_load: bool = False) -> dict:
    """{"model": {name: FlatPieces}, "optimizer": {"state": {name: {...}}, "param_groups": [...]}} in the layout of
    `get_model_state_dict` / `get_optimizer_state_dict` (names as keys, `params` of a group = its names)."""
    sd = {"model": _pieces_of(eng, "master")}
    if opt is None:
        return sd
    if hasattr(opt, "opt_name") and hasattr(opt, "step_count") and not hasattr(opt, "inner") and hasattr(opt, "hyper_for"):
        keys = _state_keys(opt)
        for u in eng.units:
            u.ensure_state(list(keys))
        per_key = {k: _pieces_of(eng, k) for k in keys}
        state = {}
        log_time = keys.get("m") == "m"
        for g in opt.param_groups:
            for n in g["param_names"]:
                st = {"step": int(opt.step_count)}
                for k, name in keys.items():
                    st[name] = per_key[k][n]
                if log_time:
                    # the scalars the per-tensor classes keep for logging (src/optim/adana.py:191-227): present so that a
                    # loader whose state has these keys finds them
                    for sk in _LOGGED_SCALARS:
                        st[sk] = torch.zeros((), dtype=torch.float32)
                state[n] = st
        groups = []
        for g in opt.param_groups:
            gg = {k: v for k, v in g.items() if k not in ("params", "param_names")}
            gg["params"] = list(g["param_names"])
            gg["param_names"] = list(g["param_names"])
            groups.append(gg)
        sd["optimizer"] = {"state": state, "param_groups": groups}
    elif not for_load:
        # any other optimizer on the engine: its own state dictionary, one entry per rank (restored on the same
        # world size only)
        from .checkpoint import _to_cpu

        sd[f"optimizer_rank{eng.rank}"] = {"blob": _to_cpu(opt.state_dict())}
    return sd


def save_engine_state(eng, opt, sharded_dir: Path):
    """Collective: every rank writes the rectangles it holds; rank 0 writes the `.metadata` index."""
    import torch.distributed as dist
    import torch.distributed.checkpoint as dcp

    SavePlanner, _ = _planners()
    sharded_dir = Path(sharded_dir)
    sharded_dir.mkdir(parents=True, exist_ok=True)
    no_dist = not (dist.is_available() and dist.is_initialized())
    dcp.save(engine_state_dict(eng, opt), checkpoint_id=str(sharded_dir), planner=SavePlanner(), no_dist=no_dist)


def load_engine_state(eng, opt, sharded_dir: Path):
    """Collective: reads, for every rectangle this rank holds now, the overlapping saved chunks (any world size)."""
    import torch.distributed as dist
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint import FileSystemReader

    _, LoadPlanner = _planners()
    sharded_dir = Path(sharded_dir)
    no_dist = not (dist.is_available() and dist.is_initialized())
    meta = FileSystemReader(str(sharded_dir)).read_metadata()
    saved_keys = set(meta.state_dict_metadata)
    target = engine_state_dict(eng, opt, for_load=True)
    fused = "optimizer" in target
    if fused and not any(k.startswith("optimizer.state.") for k in saved_keys):
        del target["optimizer"]      # a checkpoint without optimizer state (or of another optimizer family)
        fused = False
    if fused:
        # keys the checkpoint does not have (it may come from the reference: other logged scalars) are not asked for
        for n, st in target["optimizer"]["state"].items():
            for k in list(st):
                if f"optimizer.state.{n}.{k}" not in saved_keys:
                    del st[k]
        for i, g in enumerate(target["optimizer"]["param_groups"]):
            for k in list(g):
                if f"optimizer.param_groups.{i}.{k}" not in saved_keys:
                    del g[k]
    blob_key = f"optimizer_rank{eng.rank}"
    wants_blob = opt is not None and not fused and hasattr(opt, "load_state_dict") and f"{blob_key}.blob" in saved_keys
    if wants_blob:
        target[blob_key] = {"blob": None}
    dcp.load(target, checkpoint_id=str(sharded_dir), planner=LoadPlanner(), no_dist=no_dist)
    if fused:
        steps = [int(st["step"]) for st in target["optimizer"]["state"].values() if "step" in st]
        if steps:
            opt.step_count = max(steps)
        for g, sg in zip(opt.param_groups, target["optimizer"]["param_groups"]):
            for k, v in sg.items():
                if k not in ("params", "param_names"):
                    g[k] = v
    elif wants_blob:
        opt.load_state_dict(target[blob_key]["blob"])
    elif opt is not None and hasattr(opt, "inner"):
        raise RuntimeError("the state of a per-tensor optimizer under the sharded engine can only be restored on the "
                           "world size it was saved with")
    eng.refresh_from_master()
