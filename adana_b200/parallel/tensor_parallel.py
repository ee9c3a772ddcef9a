"""Tensor-parallel plans for the PyTorch path (2-D data x tensor parallel under `--tp_size`).

Each model exposes `get_tp_plan()`: block-relative module path -> "colwise" | "rowwise"
(column-parallel projections feed row-parallel ones, so one all-reduce follows each
row-parallel linear).  `apply_tensor_parallel` turns that into DTensor `parallelize_module`
calls on every block, before FSDP wraps the block on the data-parallel sub-mesh
(reference: src/distributed/fsdp.py:88-103; plans src/models/enoki.py:239-251,
src/models/qwen3.py:312-327).  Embeddings, norms and the LM head stay replicated over tp.

`FusedRowParallel` is the kernel-path building block for the row-parallel half: the GEMM whose epilogue does the
reduce-scatter over peer memory (csrc/gemm_tcgen05.cu, EPI_F32_RS), so the partial products never exist as a
tensor and the transfer overlaps the math tile by tile.
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


class FusedRowParallel:
    """Row-parallel linear + reduce-scatter in one kernel over a peer-memory plane.

    Every rank holds a K-slice of the input x [M, K/tp] and of the weight w [N, K/tp]; the full product is the sum
    of the ranks' partial products.  `__call__` leaves rank r with rows [r·M/tp, (r+1)·M/tp) of that sum (fp32), the
    sequence-parallel layout that the next norm / column-parallel linear consumes.  Two plane barriers bracket the
    launch: one after the buffers are zeroed, one before they are read."""

    def __init__(self, plane, M: int, N: int):
        import torch

        if M % plane.world != 0:
            raise ValueError(f"M={M} must divide by the {plane.world} tensor-parallel ranks")
        self.plane, self.M, self.N = plane, M, N
        self.rows = M // plane.world
        self.out = plane.alloc(self.rows * N, torch.float32).view(self.rows, N)
        self.ptrs = plane.peer_ptrs(self.out)

    def __call__(self, x_local, w_local, alpha: float = 1.0):
        from ..ops import gemm

        self.out.zero_()
        self.plane.barrier()
        gemm.linear_fwd_reduce_scatter(x_local, w_local, self.ptrs, self.rows, self.plane.rank, alpha)
        self.plane.barrier()
        return self.out
