"""Distributed backends: `single`, DDP (`nccl` / `ddp` / `gloo`) and `fsdp`.

The backend protocol is the reference's (src/distributed/backend.py:6-45): `transform_model`,
`get_context_for_microstep_forward`, `is_master_process`, `get_adjusted_args_for_process`,
`get_raw_model`, `translate_model_parameter_name_for_node`, `get_world_size`,
`clip_grad_norm_`, `all_ranks_checkpoint`, `finalize`.  What differs is what stands behind it:

  * `transform_model` attaches the kernel engine (`adana_b200.runtime.engine`) whenever the
    model has a kernel path.  `fsdp` shards the engine's state over the ranks; the DDP
    backends keep it replicated and all-reduce the flat gradient buffers.  No wrapper module
    is created, so parameter names are unchanged under every backend.
  * models without a kernel path (MoE, Llama, ...) fall back to PyTorch's own wrappers
    (`DistributedDataParallel`, FSDP2 `fully_shard`, DTensor tensor-parallel plans).
  * `gloo` runs the same engine on CPU ranks — used by the multi-process tests.
  * per-rank batch/accumulation split: `acc //= gcd(acc, N)`, `batch //= N / gcd`
    (reference src/distributed/ddp.py:24-35).
"""
from __future__ import annotations

import math
import os
from contextlib import contextmanager, nullcontext
from datetime import timedelta
from typing import List

import torch
import torch.distributed as dist

from ..parallel.comm import Comm
from ..runtime.layout import engine_supported


class DistributedBackend:
    name = "base"

    def __init__(self, args):
        self.engine = None

    # ---- protocol ---------------------------------------------------------------------------------
    def transform_model(self, model):
        raise NotImplementedError

    @contextmanager
    def get_context_for_microstep_forward(self, model, microstep_idx, gradient_accumulation_steps):
        if self.engine is not None:
            self.engine.sync_on_backward = microstep_idx == gradient_accumulation_steps - 1
            if microstep_idx == 0:
                self.engine.micro_step = 0
        yield

    def is_master_process(self) -> bool:
        return True

    def get_adjusted_args_for_process(self, args):
        return args

    def get_raw_model(self, model):
        return model

    def translate_model_parameter_name_for_node(self, parameter_name) -> List[str]:
        return [parameter_name]

    def get_world_size(self) -> int:
        return 1

    def all_ranks_checkpoint(self) -> bool:
        return False

    def clip_grad_norm_(self, parameters, max_norm, norm_type=2.0):
        """Global gradient norm; with the engine the clip coefficient stays on the device and is
        applied inside the fused optimizer step (no pass over the gradients)."""
        if self.engine is not None and self.engine.enabled and self.engine_optimizer:
            return self.engine.grad_norm_and_clip(float(max_norm))
        if self.engine is not None and self.engine.enabled:
            # engine gradients + an external (per-tensor) optimizer: scale the flat buffers
            norm = self.engine.grad_norm_and_clip(float(max_norm))
            for u in self.engine.units:
                u.grads.mul_(self.engine._clip[0])
            self.engine._clip[0] = 1.0
            return norm
        parameters = list(parameters)
        if any(getattr(p, "_adana_rank_local", False) for p in parameters) and dist.is_available() and dist.is_initialized():
            return self._clip_with_rank_local(parameters, max_norm)
        return torch.nn.utils.clip_grad_norm_(parameters, max_norm)

    @staticmethod
    def _clip_with_rank_local(parameters, max_norm):
        """Global norm when some parameters exist on one rank only (expert parallelism): the replicated gradients are
        identical everywhere and count once, the rank-local ones are summed over the ranks, so every rank derives the
        same norm and scales by the same coefficient."""
        shared = [p.grad.detach() for p in parameters if p.grad is not None and not getattr(p, "_adana_rank_local", False)]
        local = [p.grad.detach() for p in parameters if p.grad is not None and getattr(p, "_adana_rank_local", False)]
        dev = (shared or local)[0].device
        sq_local = torch.stack([g.float().pow(2).sum() for g in local]).sum() if local else torch.zeros((), device=dev)
        dist.all_reduce(sq_local)
        sq_shared = torch.stack([g.float().pow(2).sum() for g in shared]).sum() if shared else torch.zeros((), device=dev)
        total = (sq_shared + sq_local).sqrt()
        coef = torch.clamp(max_norm / (total + 1e-6), max=1.0)
        for g in shared + local:
            g.mul_(coef.to(g.dtype))
        return total

    engine_optimizer = False

    def finalize(self):
        pass

    # ---- helpers -----------------------------------------------------------------------------------
    def _maybe_attach_engine(self, model, args, sharded: bool, comm=None) -> bool:
        """Attach the kernel engine when the model has a kernel path; True when attached."""
        reason = "--no_cuda_kernels" if getattr(args, "no_cuda_kernels", False) else engine_supported(model, args)
        if reason is not None:
            if self.is_master_process():
                print(f"[engine] PyTorch path in use: {reason}")
            return False
        from ..runtime.engine import attach

        self.engine = attach(model, args, comm=comm, sharded=sharded, device=args.device)
        return True


class SingleBackend(DistributedBackend):
    name = "single"

    def transform_model(self, model):
        self._maybe_attach_engine(model, self.args, sharded=False)
        return model

    def get_adjusted_args_for_process(self, args):
        self.args = args
        return args


def _split_batch(args, ranks: int):
    eff = args.batch_size * args.acc_steps
    if eff % ranks != 0:
        raise ValueError(f"Effective batch size {eff} is not divisible by the data-parallel size {ranks}.")
    g = math.gcd(args.acc_steps, ranks)
    args.acc_steps //= g
    args.batch_size //= ranks // g
    return args


class _ProcessGroupBackend(DistributedBackend):
    sharded = False

    def __init__(self, args, pg_backend: str):
        super().__init__(args)
        self.rank = int(os.environ.get("RANK", -1))
        if self.rank == -1:
            raise RuntimeError(f"the {self.name} backend needs RANK/WORLD_SIZE (launch with torchrun)")
        self.local_rank = int(os.environ.get("LOCAL_RANK", 0))
        self.pg_backend = pg_backend
        if pg_backend == "nccl":
            assert "cuda" in args.device, "NCCL backends need CUDA devices"
            torch.cuda.set_device(self.local_rank)
        if not dist.is_initialized():
            kw = {}
            if pg_backend == "nccl":
                kw["device_id"] = torch.device("cuda", self.local_rank)
            timeout = float(os.environ.get("ADANA_PG_TIMEOUT_S", "1800"))
            dist.init_process_group(backend=pg_backend, timeout=timedelta(seconds=timeout), **kw)
        self.comm = Comm()
        self._wrapped = False

    def get_adjusted_args_for_process(self, args):
        args = _split_batch(args, self.dp_size)
        args.device = f"cuda:{self.local_rank}" if self.pg_backend == "nccl" else "cpu"
        args.seed = args.seed + self.local_rank
        self.args = args
        return args

    @property
    def dp_size(self):
        return self.get_world_size()

    def is_master_process(self) -> bool:
        return self.rank == 0

    def get_world_size(self):
        return dist.get_world_size()

    def finalize(self):
        if dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()


class DDPBackend(_ProcessGroupBackend):
    name = "ddp"

    def transform_model(self, model):
        if self._maybe_attach_engine(model, self.args, sharded=False, comm=self.comm):
            return model
        from torch.nn.parallel import DistributedDataParallel as DDP

        from ..parallel.expert_parallel import rank_local_parameters

        self._wrapped = True
        local = rank_local_parameters(model)
        if local:     # expert-parallel layers: each rank's experts are its own, not replicas to keep in step
            DDP._set_params_and_buffers_to_ignore_for_model(model, local)
        if self.pg_backend == "nccl":
            return DDP(model, device_ids=[self.local_rank])
        return DDP(model)

    @contextmanager
    def get_context_for_microstep_forward(self, model, microstep_idx, gradient_accumulation_steps):
        if self._wrapped:
            model.require_backward_grad_sync = microstep_idx == gradient_accumulation_steps - 1
            yield
        else:
            with super().get_context_for_microstep_forward(model, microstep_idx, gradient_accumulation_steps):
                yield

    def get_raw_model(self, model):
        return model.module if self._wrapped else model

    def translate_model_parameter_name_for_node(self, parameter_name):
        return [f"module.{parameter_name}"] if self._wrapped else [parameter_name]


class FSDPBackend(_ProcessGroupBackend):
    name = "fsdp"
    sharded = True

    def __init__(self, args):
        assert "cuda" in args.device or os.environ.get("ADANA_FSDP_CPU") == "1", \
            "fsdp needs CUDA devices (set ADANA_FSDP_CPU=1 to run the engine on Gloo CPU ranks)"
        super().__init__(args, "nccl" if "cuda" in args.device else "gloo")
        self.tp_size = getattr(args, "tp_size", 1)
        ws = self.get_world_size()
        if self.tp_size > 1 and ws % self.tp_size != 0:
            raise ValueError(f"world size {ws} is not divisible by tp_size {self.tp_size}")
        self._is_fsdp = True
        self._torch_fsdp = False
        self.tp_mesh = self.dp_mesh = None
        self.tp_group = self.dp_group = None
        if self.tp_size > 1:
            # rank = dp index * tp_size + tp index (the layout of a (dp, tp) device mesh); the ranks of one tp group work
            # on the same batches
            from ..data.readers import set_data_parallel_layout

            set_data_parallel_layout(ws // self.tp_size, self.rank // self.tp_size)

    @property
    def dp_size(self):
        return self.get_world_size() // self.tp_size

    def all_ranks_checkpoint(self) -> bool:
        return True

    def _make_groups(self):
        """Process groups of the 2-D layout (every rank creates every group, in the same order)."""
        ws, tp = self.get_world_size(), self.tp_size
        for i in range(ws // tp):
            ranks = list(range(i * tp, (i + 1) * tp))
            g = dist.new_group(ranks)
            if self.rank in ranks:
                self.tp_group = g
        for j in range(tp):
            ranks = list(range(j, ws, tp))
            g = dist.new_group(ranks)
            if self.rank in ranks:
                self.dp_group = g

    def transform_model(self, model):
        if self.tp_size == 1:
            if self._maybe_attach_engine(model, self.args, sharded=True, comm=self.comm):
                return model
            return self._torch_fully_shard(model)
        # dp x tp on the kernel engine: flat shards over the data-parallel group of this tp index, heads and hidden units
        # cut over the tp group (parallel/tensor_parallel.py); models without a kernel path take DTensor plans + FSDP2
        from ..parallel.tensor_parallel import check_divisible
        from ..runtime.layout import engine_supported

        if not getattr(self.args, "no_cuda_kernels", False) and engine_supported(model, self.args) is None:
            check_divisible(model, self.tp_size)
            self._make_groups()
            from ..runtime.engine import attach

            self.engine = attach(model, self.args, comm=Comm(self.dp_group), sharded=True, device=self.args.device,
                                 tp_group=self.tp_group)
            return model
        return self._torch_fully_shard(model)

    # -- library fallback: FSDP2 (+ DTensor tensor parallelism) for models without a kernel path ---------
    def _torch_fully_shard(self, model):
        from torch.distributed.device_mesh import init_device_mesh
        from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

        from ..parallel.expert_parallel import rank_local_parameters

        if rank_local_parameters(model):
            # FSDP2 shards every parameter as one tensor that all ranks hold alike; each rank's own experts are not that
            raise ValueError("expert-parallel layers cannot be sharded by torch FSDP2: pass --no_expert_parallel, or use "
                             "--distributed_backend nccl (data parallelism with the experts split over the ranks)")
        self._torch_fsdp = True
        dev_type = "cuda" if self.pg_backend == "nccl" else "cpu"
        mp = MixedPrecisionPolicy(param_dtype=torch.float32, reduce_dtype=torch.bfloat16)
        kw = {"mp_policy": mp}
        if self.tp_size > 1:
            from ..parallel.tensor_parallel import apply_tensor_parallel

            mesh = init_device_mesh(dev_type, (self.dp_size, self.tp_size), mesh_dim_names=("dp", "tp"))
            self.dp_mesh, self.tp_mesh = mesh["dp"], mesh["tp"]
            apply_tensor_parallel(model, self.tp_mesh)
            kw["mesh"] = self.dp_mesh
        for blk in model.transformer.h:
            fully_shard(blk, **kw)
        fully_shard(model, **kw)
        return model

    @contextmanager
    def get_context_for_microstep_forward(self, model, microstep_idx, gradient_accumulation_steps):
        if self._torch_fsdp:
            model.set_requires_gradient_sync(microstep_idx == gradient_accumulation_steps - 1)
            yield
        else:
            with super().get_context_for_microstep_forward(model, microstep_idx, gradient_accumulation_steps):
                yield

    def clip_grad_norm_(self, parameters, max_norm, norm_type=2.0):
        if not self._torch_fsdp:
            return super().clip_grad_norm_(parameters, max_norm, norm_type)
        from torch.distributed.tensor import DTensor

        params = [p for p in parameters if p.grad is not None]
        if not params:
            return torch.tensor(0.0)
        norms = []
        for p in params:
            g = p.grad.detach()
            n = g.full_tensor().norm(norm_type) if (isinstance(g, DTensor) and self.tp_size > 1) else g.norm(norm_type)
            if isinstance(n, DTensor):
                n = n.full_tensor()
            norms.append(n)
        total = torch.norm(torch.stack(norms), norm_type)
        coef = torch.clamp(max_norm / (total + 1e-6), max=1.0)
        for p in params:
            p.grad.detach().mul_(coef)
        return total


BACKEND_TYPE_TO_MODULE_MAP = {
    "nccl": lambda args: DDPBackend(args, "nccl"),
    "ddp": lambda args: DDPBackend(args, "nccl"),
    "gloo": lambda args: DDPBackend(args, "gloo"),
    "fsdp": FSDPBackend,
    "single": SingleBackend,
    None: SingleBackend,
}


def make_backend_from_args(args) -> DistributedBackend:
    return BACKEND_TYPE_TO_MODULE_MAP[args.distributed_backend](args)


def registered_backends():
    return BACKEND_TYPE_TO_MODULE_MAP.keys()
