"""Tensor-parallel plans for the PyTorch path (2-D data x tensor parallel under `--tp_size`).

Each model exposes `get_tp_plan()`: block-relative module path -> "colwise" | "rowwise"
(column-parallel projections feed row-parallel ones, so one all-reduce follows each
row-parallel linear).  `apply_tensor_parallel` turns that into DTensor `parallelize_module`
calls on every block, before FSDP wraps the block on the data-parallel sub-mesh
(reference: src/distributed/fsdp.py:88-103; plans src/models/enoki.py:239-251,
src/models/qwen3.py:312-327).  Embeddings, norms and the LM head stay replicated over tp.
"""
from __future__ import annotations


def apply_tensor_parallel(model, tp_mesh) -> None:
    from torch.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel, parallelize_module

    plan_fn = getattr(type(model), "get_tp_plan", None)
    if plan_fn is None:
        raise ValueError(f"Model {type(model).__name__} does not define get_tp_plan(); tensor parallelism unavailable")
    styles = {"colwise": ColwiseParallel, "rowwise": RowwiseParallel}
    plan = {path: styles[kind]() for path, kind in plan_fn().items()}
    n_head = model.config.n_head
    tp = tp_mesh.size()
    if n_head % tp != 0:
        raise ValueError(f"n_head={n_head} is not divisible by tp_size={tp}")
    for blk in model.transformer.h:
        parallelize_module(blk, tp_mesh, plan)
