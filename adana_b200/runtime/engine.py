"""Kernel engine: flat sharded state, manual forward/backward over the sm_100a ops, gradient
reduction and the fused optimizer step.

What the engine owns, per unit (one per transformer block + a root unit):

    master   fp32 [padded / world]   this rank's shard of the parameters (world = 1: everything)
    m, v, τ  fp32 [padded / world]   optimizer moments of that shard
    grads    fp32 [padded]           full-size main-gradient buffer; weight-gradient GEMMs
                                     accumulate into it across micro-steps
    weights  bf16 [padded]           compute copy of ALL parameters of the unit, resident

The bf16 copies stay resident (a 2.5 B-parameter model is 5 GB of a 180 GB device), so the
parameters cross NVLink once per optimizer step — the all-gather of the freshly updated bf16
shards, unit by unit, overlapping the first forward of the next step — instead of twice per
micro-step as in a reshard-after-forward design.  Gradients are reduce-scattered per unit as
soon as the unit's backward finishes on the last micro-step (overlapping the rest of the
backward), the squared-norm partials are produced from the reduced shards, one scalar
all-reduce gives the clip coefficient on the device, and one fused kernel per unit range
applies clip + update + weight decay and writes the bf16 shard for the next gather.

Modes: `sharded` (the `fsdp` backend; state partitioned, ZeRO-style) and replicated (the
`nccl`/`gloo` DDP backends; gradients all-reduced, every rank updates everything).  The math
matches the reference's FSDP2 / DDP training step (src/distributed/fsdp.py:88-173,
src/distributed/ddp.py:46-59, src/optim/base.py:234-294).

`attach(model, ...)` wires the engine into a model: `model(idx, targets=...)` then runs the
kernel path and `loss.backward()` runs the manual backward through a one-node autograd bridge.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from ..ops import _lib
from ..ops import misc as M
from ..ops import optim as O
from ..optim.logtime import wd_multiplier
from ..parallel.comm import Comm, wait
from . import blocks as BK
from .layout import UnitLayout, build_layouts, engine_supported

FUSED_OPTS = {"adana": (O.KIND_ADANA, False), "dana-mk4": (O.KIND_ADANA, True),
              "dana-star": (O.KIND_DANA_STAR, False), "dana-star-mk4": (O.KIND_DANA_STAR, True),
              "adamw": (O.KIND_ADAMW, False), "adamw-decaying-wd": (O.KIND_ADAMW_IWD, False),
              "ademamix": (O.KIND_ADEMAMIX, False), "ademamix-decaying-wd": (O.KIND_ADEMAMIX_IWD, False)}
_THREE_STATE = (O.KIND_DANA_STAR, O.KIND_ADEMAMIX, O.KIND_ADEMAMIX_IWD)     # kinds with a third moment buffer ("tau")


class _Bridge(torch.autograd.Function):
    """One autograd node for the whole model: backward() runs the engine's manual backward."""

    @staticmethod
    def forward(ctx, anchor, engine, loss):
        ctx.engine = engine
        return loss.detach().clone()

    @staticmethod
    def backward(ctx, grad_out):
        ctx.engine._backward(grad_out)
        return None, None, None


class Unit:
    def __init__(self, layout: UnitLayout, world: int, rank: int, sharded: bool, device, cdt, plane=None,
                 resident_weights: bool = True, reduce_bf16: bool = False):
        self.layout = layout
        self.slices = {}     # gathered mode: key -> (slice buffer, row_starts, flat offset, rows, cols)
        self.segments = []   # gathered mode: (flat_lo, flat_hi, owner rank, address of the owner's slice buffer)
        self.plane = plane
        self.padded = layout.padded
        self.shard_len = layout.padded // world if sharded else layout.padded
        self.shard_off = rank * self.shard_len if sharded else 0
        f32 = dict(dtype=torch.float32, device=device)
        self.master = torch.zeros(self.shard_len, **f32)
        self.grads = plane.alloc(self.padded, torch.float32) if plane is not None else torch.zeros(self.padded, **f32)
        # wire copy of the gradients for a bf16 reduce (peers read it; sums stay fp32)
        self.grads16 = plane.alloc(self.padded, torch.bfloat16) if (plane is not None and reduce_bf16) else None
        self.grad_shard = torch.zeros(self.shard_len, **f32) if (sharded and world > 1) else self.grads
        self.low_precision = cdt != torch.float32
        if self.low_precision and not resident_weights:
            # gathered mode: no rank holds the unit's bf16 weights in one piece (see Engine._make_slices)
            self.weights = None
            self.w_shard = None
        elif self.low_precision:
            self.weights = (plane.alloc(self.padded, cdt) if plane is not None
                            else torch.zeros(self.padded, dtype=cdt, device=device))
            if plane is not None:      # peers store into `weights` directly: my shard is a slice of it
                self.w_shard = self.weights[self.shard_off:self.shard_off + self.shard_len]
            else:
                self.w_shard = (torch.zeros(self.shard_len, dtype=cdt, device=device)
                                if (sharded and world > 1) else self.weights)
        else:
            # fp32 compute: the master buffer is the compute buffer when it is complete
            self.weights = self.master if self.shard_len == self.padded else torch.zeros(self.padded, **f32)
            self.w_shard = self.master
        self.state: Dict[str, torch.Tensor] = {}
        self.grad_work = None
        self.gather_work = None
        self.grads_dirty = False
        # 1-D parameters are consumed in fp32 by the norm kernels
        one_d = [s for s in layout.slots if len(s.shape) == 1]
        self.small_off = min((s.offset for s in one_d), default=layout.numel)
        assert all(len(s.shape) == 1 for s in layout.slots if s.offset >= self.small_off)
        self.small_len = layout.numel - self.small_off
        self.small_f32: Optional[torch.Tensor] = None

    def ensure_state(self, names):
        for n in names:
            if n not in self.state:
                self.state[n] = torch.zeros_like(self.master)

    def view(self, flat: torch.Tensor, slot) -> torch.Tensor:
        return flat[slot.offset: slot.offset + slot.numel].view(slot.shape)


@dataclass
class EngineConfig:
    acc_steps: int = 1
    grad_clip: float = 0.0
    z_loss_coeff: float = 0.0
    hoyer_loss_coeff: float = 0.0
    activation_checkpointing: bool = False
    checkpoint_every_n: int = 1
    reduce_dtype: str = "float32"
    log_diagnostics: bool = False


class Engine:
    def __init__(self, model, cfg, comm: Optional[Comm] = None, sharded: bool = True,
                 device=None, compute_dtype: Optional[torch.dtype] = None, tp_group=None):
        reason = engine_supported(model, cfg)
        if reason is not None:
            raise ValueError(f"kernel engine unavailable: {reason}")
        self.model = model
        self.cfg = cfg
        self.comm = comm or Comm()
        self.world, self.rank = self.comm.world, self.comm.rank
        self.sharded = sharded and self.world > 1
        self.device = torch.device(device if device is not None else next(model.parameters()).device)
        if compute_dtype is None:
            compute_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32,
                             "float16": torch.bfloat16}[getattr(cfg, "dtype", "bfloat16")]
            if self.device.type == "cpu" and getattr(cfg, "dtype", "float32") == "float32":
                compute_dtype = torch.float32
        self.cdt = compute_dtype
        self.ecfg = EngineConfig(
            acc_steps=getattr(cfg, "acc_steps", 1), grad_clip=getattr(cfg, "grad_clip", 0.0),
            z_loss_coeff=getattr(cfg, "z_loss_coeff", 0.0), hoyer_loss_coeff=getattr(cfg, "hoyer_loss_coeff", 0.0),
            activation_checkpointing=getattr(cfg, "activation_checkpointing", False),
            checkpoint_every_n=getattr(cfg, "checkpoint_every_n", 1),
            # the dtype gradients cross the links in (sums are always fp32); bf16 is what the reference's FSDP uses
            # (src/distributed/fsdp.py:39-43).  fp32 compute keeps fp32 on the wire.
            reduce_dtype="float32" if self.cdt == torch.float32 else getattr(cfg, "reduce_dtype", "bfloat16"))
        self.loss_scale = 1.0 / max(1, self.ecfg.acc_steps)
        self.enabled = True
        if getattr(cfg, "attention", "auto") != "auto":
            from ..ops import attention as _att

            _att.set_mode(cfg.attention)

        # tensor parallelism: `comm` is then the data-parallel group of this rank's tp index, and the module tree is
        # cut down to this rank's heads and hidden units before the flat layout is made
        self.tp = None
        if tp_group is not None and torch.distributed.get_world_size(tp_group) > 1:
            from ..parallel.tensor_parallel import TensorParallelGroup, shard_model_for_tp

            with torch.no_grad():
                for p in model.parameters():        # every rank cuts the same initialisation: global rank 0's
                    torch.distributed.broadcast(p.data, src=0)
            self.tp = TensorParallelGroup(tp_group, self.device, self.cdt)
            self.tp.cut = shard_model_for_tp(model, self.tp.rank, self.tp.size)
        self.layouts = build_layouts(model, self.world if self.sharded else 1)
        plane = self._make_plane()
        # the sharded engine runs every collective on the plane; a replicated (data-parallel) engine only the
        # gradient all-reduce
        self.plane = plane if self.sharded else None
        self.ar_plane = plane if not self.sharded else None
        self.reduce_bf16 = plane is not None and self.ecfg.reduce_dtype == "bfloat16"
        self.reduce_seq = 0
        # `--fsdp_weights gathered`: the block matrices are never all-gathered.  With the peer-memory plane every
        # rank keeps only its row slice of each matrix and the GEMMs fetch B tiles from the owners; without it
        # (one GPU) the slices are views of the resident matrix, which exercises the same GEMM path.
        self.gathered = (getattr(cfg, "fsdp_weights", "resident") == "gathered" and self.device.type == "cuda"
                         and self.cdt == torch.bfloat16 and getattr(model, "arch", "") == "enoki"
                         and not getattr(cfg, "moe", False) and self.tp is None)
        split = self.gathered and self.plane is not None
        self.units: List[Unit] = [Unit(l, self.world, self.rank, self.sharded, self.device, self.cdt, plane,
                                       resident_weights=not (split and l.name != "root"), reduce_bf16=self.reduce_bf16)
                                  for l in self.layouts]
        self._unit_index = {u.layout.name: i for i, u in enumerate(self.units)}
        self.spec = self._block_spec()
        self.tied = False
        # plain cross-entropy without the z term and without auxiliary outputs (src/models/llama.py:197-215)
        self.plain_loss = getattr(model, "arch", "") == "llama"
        if split:
            self._make_slices()
        self.freqs = model.freqs_cis.to(self.device).contiguous()
        self._anchor = torch.zeros((), device=self.device, requires_grad=True)
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._clip = torch.ones(2, dtype=torch.float32, device=self.device)
        self._diag = torch.zeros(4, dtype=torch.float32, device=self.device)
        self._pending = None
        self.micro_step = 0            # micro-steps accumulated since the last optimizer step
        self.sync_on_backward = None   # None: automatic (last of acc_steps); bool: forced by the backend
        self.opt_step_count = 0
        # a replicated engine under an optimizer that is not its own hands out averaged gradients (the fused step
        # folds the 1 / world into its update instead); set by `optim.registry.build_optimizer`
        self.average_on_sync = False
        self._averaged = False
        # report the Hoyer value of the embeddings with every forward even when it does not enter the loss, as the
        # reference's models do; the training loop switches it off on iterations that log nothing
        self.report_aux = True
        self.last_grad_norm = None
        self.launches = 0
        self._meter_pairs = []

        self._load_from_module()
        self._bind_views()
        self._sync_small()
        self._rebind_module_params()

    # ---------------------------------------------------------------------------------------------
    # construction helpers
    # ---------------------------------------------------------------------------------------------
    def _make_plane(self):
        """Peer-memory data plane for the sharded engine on GPUs (`--fsdp_comm auto|p2p`); None selects
        torch.distributed collectives (NCCL / Gloo)."""
        want = getattr(self.cfg, "fsdp_comm", "auto")
        if self.world < 2 or self.device.type != "cuda" or self.cdt == torch.float32 or want == "nccl":
            return None
        if self.world > 8 or not _lib.has("adana_p2p_reduce_scatter_flag"):
            return None
        # per unit: fp32 gradients (4) + bf16 weights (2) + bf16 wire copy of the gradients (2) + fp32 norm weights
        # plus 64 KiB for small tables of optimizers that talk over the plane (distributed Muon's partial norms)
        nbytes = sum(l.padded * 8 + l.numel * 4 + 4096 for l in self.layouts) + (1 << 16)
        plane, err = None, None
        try:
            from ..parallel.p2p import P2PPlane

            plane = P2PPlane.create(nbytes, self.device, group=self.comm.group)
        except Exception as e:
            err = e
        # every rank must take the same plane: one rank without peer memory sends all of them to NCCL
        ok = torch.tensor([0.0 if plane is None else 1.0], device=self.device)
        self.comm.all_reduce_sum(ok)
        if int(ok.item()) == self.world:
            return plane
        if want == "p2p":
            raise RuntimeError(f"--fsdp_comm p2p: the peer-memory plane could not be set up on every rank ({err})")
        if self.rank == 0:
            print(f"[engine] peer-memory plane unavailable on {self.world - int(ok.item())} rank(s) ({err}); "
                  f"using NCCL collectives")
        if plane is not None:
            del plane
        return None

    # ---- gathered weights ----------------------------------------------------------------------------------
    _MATS = (("qkv", "attn.c_attn.weight"), ("o", "attn.c_proj.weight"), ("fc", "mlp.c_fc.weight"),
             ("down", "mlp.c_proj.weight"))

    def _make_slices(self):
        """Row slices of every block matrix in the symmetric arena, cut on whole 128-row tiles; rank r keeps rows
        [row_starts[r], row_starts[r+1]).  `segments` maps flat ranges of the unit to (owner, owner's buffer)."""
        from ..ops.gemm import tile_aligned_row_starts

        for u in self.units:
            if u.weights is not None:
                continue
            for key, suffix in self._MATS:
                sl = u.layout.slot(suffix)
                rows, cols = sl.shape
                starts = tile_aligned_row_starts(rows, self.world)
                if any(b <= a for a, b in zip(starts, starts[1:])):
                    raise ValueError(f"--fsdp_weights gathered: {sl.name} has fewer 128-row tiles than ranks")
                most = max(b - a for a, b in zip(starts, starts[1:]))
                buf = self.plane.alloc(most * cols, self.cdt)
                ptrs = self.plane.peer_ptrs(buf)
                u.slices[key] = (buf, starts, sl.offset, rows, cols, ptrs)
                for r in range(self.world):
                    u.segments.append((sl.offset + starts[r] * cols, sl.offset + starts[r + 1] * cols, r, int(ptrs[r])))
            u.segments.sort()

    def _fill_slices(self, u: Unit, full: torch.Tensor):
        """Copy this rank's rows of every matrix out of a full copy of the unit's parameters."""
        for key, (buf, starts, off, rows, cols, _) in u.slices.items():
            a, b = starts[self.rank], starts[self.rank + 1]
            buf[:(b - a) * cols].copy_(full[off + a * cols: off + b * cols])

    def _block_spec(self) -> BK.BlockSpec:
        m, c = self.model, self.cfg
        hd = m.head_dim
        tp = self.tp.size if self.tp is not None else 1        # (the MLP width is read off the already cut matrices)
        if m.arch == "enoki":
            mlp = m.transformer.h[0].mlp.c_fc.weight.shape[0]
            qk_kind = BK.R.NONORM if getattr(c, "no_qknorm", False) else BK.R.LAYERNORM
            return BK.BlockSpec(d=c.n_embd, n_head=c.n_head // tp, n_kv_head=c.n_head // tp, hd=hd, mlp=mlp,
                                mlp_kind="gelu", norm_kind=BK.N.LAYERNORM, qk_kind=qk_kind, gate=False,
                                eps=1e-5, qk_eps=1e-5, scale=float(getattr(c, "residual_stream_scalar", 1.0)),
                                seq_len=c.sequence_length)
        if m.arch == "llama":
            # RMSNorm, fused q|k|v, RoPE without a per-head norm, SwiGLU (w1 = gate, w2 = up), tied embeddings
            return BK.BlockSpec(d=c.n_embd, n_head=c.n_head // tp, n_kv_head=c.n_head // tp, hd=hd,
                                mlp=m.transformer.h[0].mlp.w1.weight.shape[0], mlp_kind="swiglu", norm_kind=BK.N.RMSNORM,
                                qk_kind=BK.R.NONORM, gate=False, eps=float(getattr(c, "rmsnorm_eps", 1e-5)),
                                qk_eps=1e-5, scale=1.0, seq_len=c.sequence_length)
        blk = m.transformer.h[0]
        rms = getattr(c, "normalization_layer_type", "rmsnorm") == "rmsnorm"
        eps = float(getattr(c, "rmsnorm_eps", 1e-5)) if rms else 1e-5
        qk_kind = BK.R.NONORM if getattr(c, "no_qknorm", False) else (BK.R.RMSNORM if rms else BK.R.LAYERNORM)
        return BK.BlockSpec(d=c.n_embd, n_head=c.n_head // tp, n_kv_head=blk.attn.n_kv_head // tp, hd=hd,
                            mlp=blk.mlp.gate_proj.weight.shape[0], mlp_kind="swiglu",
                            norm_kind=BK.N.RMSNORM if rms else BK.N.LAYERNORM, qk_kind=qk_kind,
                            gate=blk.attn.gate, eps=eps, qk_eps=eps,
                            scale=float(getattr(c, "residual_stream_scalar", 1.0)), seq_len=c.sequence_length)

    def _load_from_module(self):
        """Copy the module's (full, fp32) parameters into master shards and compute buffers."""
        params = dict(self.model.named_parameters())
        with torch.no_grad():
            for u in self.units:
                full = torch.zeros(u.padded, dtype=torch.float32, device=self.device)
                for s in u.layout.slots:
                    full[s.offset:s.offset + s.numel].copy_(params[s.name].detach().reshape(-1).float())
                if self.world > 1:
                    # every rank starts from rank 0's initialisation, whatever its own seed was
                    self.comm.broadcast(full, src=0)
                u.master.copy_(full[u.shard_off:u.shard_off + u.shard_len])
                if u.weights is None:
                    self._fill_slices(u, full)
                elif u.weights.data_ptr() != u.master.data_ptr():
                    u.weights.copy_(full)
                del full

    def _bind_views(self):
        """Per-unit dictionaries of weight / gradient views used by the block functions."""
        sp = self.spec
        for u in self.units:
            lay = u.layout
            if u.shard_len == u.padded:
                u.small_f32 = u.master[u.small_off:u.small_off + u.small_len]
            elif self.plane is not None:
                u.small_f32 = self.plane.alloc(max(u.small_len, 1), torch.float32)[:u.small_len]
            else:
                u.small_f32 = torch.zeros(u.small_len, dtype=torch.float32, device=self.device)

            def small(slot, u=u):
                o = slot.offset - u.small_off
                return u.small_f32[o:o + slot.numel]

            W, Gd = {}, {}
            if lay.name == "root":
                for key, suffix in (("lm_head", "lm_head.weight"), ("wte", "transformer.wte.weight")):
                    if not lay.has(suffix):
                        continue
                    sl = lay.slot(suffix)
                    W[key], Gd[key] = u.view(u.weights, sl), u.view(u.grads, sl)
                self.tied = "lm_head" not in W
                if self.tied:                   # one table serves as embedding and as LM head: both gradients meet in it
                    W["lm_head"], Gd["lm_head"] = W["wte"], Gd["wte"]
                sl = lay.slot("transformer.ln_f.weight")
                W["ln_f"], Gd["ln_f"] = small(sl), u.view(u.grads, sl)
            else:
                def fused(suffixes, rows_cols):
                    first = lay.slot(suffixes[0])
                    off = first.offset
                    for sfx in suffixes:
                        sl = lay.slot(sfx)
                        assert sl.offset == off, f"{sl.name} is not adjacent in the flat layout"
                        off += sl.numel
                    n = off - first.offset
                    r, c = rows_cols
                    assert n == r * c
                    gview = u.grads[first.offset:first.offset + n].view(r, c)
                    if u.weights is None:
                        return None, gview                 # gathered: the weight entry is set below
                    return u.weights[first.offset:first.offset + n].view(r, c), gview
                if self.model.arch == "llama":
                    W["qkv"], Gd["qkv"] = fused(["attn.c_attn.weight"], (sp.proj_out, sp.d))
                    W["o"], Gd["o"] = fused(["attn.c_proj.weight"], (sp.d, sp.n_head * sp.hd))
                    W["fc"], Gd["fc"] = fused(["mlp.w1.weight", "mlp.w2.weight"], (2 * sp.mlp, sp.d))
                    W["down"], Gd["down"] = fused(["mlp.c_proj.weight"], (sp.d, sp.mlp))
                    qn = kn = "attn.no_such_norm.weight"
                elif self.model.arch == "enoki":
                    W["qkv"], Gd["qkv"] = fused(["attn.c_attn.weight"], (sp.proj_out, sp.d))
                    W["o"], Gd["o"] = fused(["attn.c_proj.weight"], (sp.d, sp.n_head * sp.hd))
                    W["fc"], Gd["fc"] = fused(["mlp.c_fc.weight"], (sp.mlp, sp.d))
                    W["down"], Gd["down"] = fused(["mlp.c_proj.weight"], (sp.d, sp.mlp))
                    qn, kn = "attn.q_layernorm.weight", "attn.k_layernorm.weight"
                    if self.gathered:
                        self._bind_gathered(u, W)
                else:
                    W["qkv"], Gd["qkv"] = fused(["attn.q_proj.weight", "attn.k_proj.weight", "attn.v_proj.weight"],
                                                (sp.proj_out, sp.d))
                    W["o"], Gd["o"] = fused(["attn.o_proj.weight"], (sp.d, sp.n_head * sp.hd))
                    W["fc"], Gd["fc"] = fused(["mlp.gate_proj.weight", "mlp.up_proj.weight"], (2 * sp.mlp, sp.d))
                    W["down"], Gd["down"] = fused(["mlp.down_proj.weight"], (sp.d, sp.mlp))
                    qn, kn = "attn.q_norm.weight", "attn.k_norm.weight"
                for key, suffix in (("ln_1", "ln_1.weight"), ("ln_2", "ln_2.weight"), ("q_norm", qn), ("k_norm", kn)):
                    if lay.has(suffix):
                        sl = lay.slot(suffix)
                        W[key], Gd[key] = small(sl), u.view(u.grads, sl)
            u.W, u.Gd = W, Gd

    def _bind_gathered(self, u: Unit, W: dict):
        """Replace the four block matrices of `W` by `ShardedWeight`s."""
        from ..ops.gemm import ShardedWeight, tile_aligned_row_starts

        for idx, (key, _) in enumerate(self._MATS):
            if u.weights is None:      # true row slices, one per rank, addressed through peer pointers
                buf, starts, off, rows, cols, ptrs = u.slices[key]
                W[key] = ShardedWeight(list(ptrs), starts, rows, cols, local=None, me=self.rank)
            else:                      # one process: up to 8 virtual slices that are views of the resident matrix
                w = W[key]
                rows, cols = w.shape
                k = max(1, min(8, rows // 128))
                starts = tile_aligned_row_starts(rows, k)
                views = [w[a:b] for a, b in zip(starts, starts[1:])]
                W[key] = ShardedWeight(views, starts, rows, cols, local=views, me=idx % k)

    def _rebind_module_params(self):
        """Point the module's parameters at the engine's storage (or release them when sharded)."""
        params = dict(self.model.named_parameters())
        with torch.no_grad():
            for u in self.units:
                for s in u.layout.slots:
                    p = params[s.name]
                    if u.shard_len == u.padded:
                        p.data = u.view(u.master, s)
                        p.grad = u.view(u.grads, s)
                    else:
                        p.data = torch.empty(0, dtype=torch.float32, device=self.device)
                        p.grad = None
        self.model._engine = self
        replicated = [params[s.name] for u in self.units if u.shard_len == u.padded for s in u.layout.slots]
        self._first_param = replicated[0] if replicated else None

    # ---------------------------------------------------------------------------------------------
    # forward / backward
    # ---------------------------------------------------------------------------------------------
    def handles(self, model, idx, targets, get_logits) -> bool:
        return self.enabled and targets is not None and not get_logits

    def _wait_unit(self, u: Unit):
        if u.gather_work is not None:
            e0 = self._meter_begin()
            wait(u.gather_work)
            u.gather_work = None
            self._meter_end(e0)

    def _sync_small(self):
        """Sharded mode: norm weights are consumed in fp32, so their master values (owned by
        whichever rank's shard covers them) are exchanged exactly with one small all-reduce of
        a zero-padded buffer instead of being read back from the bf16 compute copy."""
        if not (self.sharded and self.world > 1):
            return
        if self.plane is not None:
            for u in self.units:
                lo, hi = u.shard_off, u.shard_off + u.shard_len
                a, b = max(u.small_off, lo), min(u.small_off + u.small_len, hi)
                if a < b:
                    self.plane.push_f32(u.master[a - lo:b - lo], u.small_f32, a - u.small_off)
            self.plane.barrier()
            return
        total = sum(u.small_len for u in self.units)
        if self._small_all is None or self._small_all.numel() != total:
            self._small_all = torch.zeros(total, dtype=torch.float32, device=self.device)
        buf = self._small_all
        buf.zero_()
        pos = 0
        for u in self.units:
            lo, hi = u.shard_off, u.shard_off + u.shard_len
            a, b = max(u.small_off, lo), min(u.small_off + u.small_len, hi)
            if a < b:
                buf[pos + a - u.small_off: pos + b - u.small_off].copy_(u.master[a - lo:b - lo])
            pos += u.small_len
        self.comm.all_reduce_sum(buf)
        pos = 0
        for u in self.units:
            u.small_f32.copy_(buf[pos:pos + u.small_len])
            pos += u.small_len

    _small_all = None

    def forward(self, idx, targets, compute_accuracy: bool = False, sample_targets: bool = False):
        """`sample_targets`: ignore `targets` and draw every position's label from the model's own predictive
        distribution, plain cross-entropy without the z term: the extra backward of Sophia's Hessian estimate
        (src/optim/base.py:268-284), which the reference runs on full logits."""
        model, sp, ecfg = self.model, self.spec, self.ecfg
        need_grad = model.training and torch.is_grad_enabled()
        B, S = idx.shape
        T = B * S
        assert S <= self.cfg.sequence_length
        idx_flat = idx.reshape(-1)
        root = self.units[-1]
        self._wait_unit(root)
        x = M.embedding_fwd(idx_flat, root.W["wte"])
        x0 = x
        saved: List = []
        ckpt = ecfg.activation_checkpointing and need_grad
        for i, u in enumerate(self.units[:-1]):
            self._wait_unit(u)
            keep = need_grad and not (ckpt and i % ecfg.checkpoint_every_n == 0)
            x_in = x
            x, sv = BK.block_forward(x, u.W, sp, self.freqs, B, S, self.cdt, need_grad=keep, tp=self.tp)
            saved.append(sv if keep else ({"x_only": x_in} if need_grad else None))
        acc = self.micro_step > 0
        out, dx, dx_lp = BK.head_forward_backward(
            x, None if sample_targets else targets, root.W, root.Gd, sp.norm_kind, sp.eps,
            0.0 if (sample_targets or self.plain_loss) else ecfg.z_loss_coeff, self.loss_scale, self.cdt, need_grad, acc)
        loss = out["loss"]
        aux = {"z_loss": out["z"]}
        hoyer_grad = None
        if self.plain_loss:
            aux = {}                # (this model family reports no auxiliary terms)
        elif ecfg.hoyer_loss_coeff != 0.0:
            hv, hoyer_grad = BK.hoyer_value_and_grad(x0, ecfg.hoyer_loss_coeff, self.loss_scale, need_grad)
            aux["hoyer_loss"] = hv
            loss = loss + ecfg.hoyer_loss_coeff * hv
        elif self.report_aux or not need_grad:
            # reported even when it does not enter the loss, as the reference's models do (src/models/enoki.py:341-343):
            # two reductions over [T, d], skipped on training iterations whose outputs nobody reads
            with torch.no_grad():
                aux["hoyer_loss"] = BK.hoyer_value_and_grad(x0, 0.0, self.loss_scale, False)[0]
        accuracy = (out["correct"] / T) if compute_accuracy else None
        if need_grad:
            self._pending = dict(dx=dx, dx_lp=dx_lp, saved=saved, idx=idx_flat, B=B, S=S,
                                 hoyer_grad=hoyer_grad, acc=acc)
            loss = _Bridge.apply(self._anchor, self, loss)
        return {"logits": None, "loss": loss, "aux_losses": aux, "router_logits": None, "accuracy": accuracy}

    def _backward(self, grad_out):
        pend = self._pending
        if pend is None:
            raise RuntimeError("engine backward called without a pending forward")
        self._pending = None
        sp = self.spec
        dx, dx_lp, saved, B, S, acc = pend["dx"], pend["dx_lp"], pend["saved"], pend["B"], pend["S"], pend["acc"]
        sync = self.sync_on_backward
        if sync is None:
            sync = (self.micro_step + 1) >= self.ecfg.acc_steps
        root = self.units[-1]
        if self.micro_step == 0:
            self._averaged = False
            if (self.plane or self.ar_plane) is not None:
                self._sumsq.zero_()  # the reductions of this optimizer step accumulate their squared-norm partials here
        with torch.no_grad():
            for i in range(len(self.units) - 2, -1, -1):
                u = self.units[i]
                sv = saved[i]
                saved[i] = None
                if "x_only" in sv:  # activation checkpoint: rebuild the block's activations
                    _, sv = BK.block_forward(sv["x_only"], u.W, sp, self.freqs, B, S, self.cdt, need_grad=True, tp=self.tp)
                BK.block_backward(dx, dx_lp, sv, u.W, u.Gd, sp, self.freqs, B, S, acc, tp=self.tp)
                u.grads_dirty = True
                del sv
                if sync:
                    self._reduce_unit(u)
            if pend["hoyer_grad"] is not None:
                dx += pend["hoyer_grad"]
            if not acc and not self.tied:        # (a tied table already holds the LM head's gradient of this micro-step)
                root.Gd["wte"].zero_()
            M.embedding_bwd(pend["idx"], dx, root.Gd["wte"])
            root.grads_dirty = True
            if sync and self.tp is not None and self.device.type == "cuda":
                # the embedding gradient is summed with atomics, in an order that differs from run to run: the tp ranks
                # (which hold this replicated table) all continue with tp rank 0's sum, so the table never drifts apart
                self.tp.broadcast_(root.Gd["wte"])
            if sync:
                self._reduce_unit(root)
        self.micro_step += 1

    # ---------------------------------------------------------------------------------------------
    # gradient reduction, clipping, optimizer
    # ---------------------------------------------------------------------------------------------
    def _reduce_unit(self, u: Unit):
        """Start the reduction of a unit's gradients (its backward has been enqueued on the current stream)."""
        if self.world == 1:
            return
        plane = self.plane or self.ar_plane
        if plane is not None:
            # This rank's copy is complete once the kernels enqueued so far have run: round it to the wire dtype,
            # then raise the unit's flag on every rank.  The pulling kernel (side stream) waits, bounded, for the flags
            # of all ranks: no barrier, so a fast rank is never stopped in the middle of its backward by a slow one.
            idx = self._unit_index[u.layout.name]
            seq = self.reduce_seq + 1
            src = u.grads
            if u.grads16 is not None:
                O.cast_f32_to_bf16(u.grads, u.grads16)
                src = u.grads16
            plane.signal_unit(idx, seq)
            ev = torch.cuda.Event()
            ev.record()
            with torch.cuda.stream(plane.stream):
                plane.stream.wait_event(ev)
                if self.sharded:
                    plane.reduce_scatter_unit(src, u.shard_off, u.grad_shard, self._sumsq, idx, seq)
                else:
                    n = -(-u.padded // (8 * self.world)) * 8          # this rank's slice, a multiple of 8 elements
                    off = min(self.rank * n, u.padded)
                    plane.all_reduce_unit(src, u.grads, off, min(n, u.padded - off), idx, seq, sumsq=self._sumsq)
            u.grad_work = None
            self._plane_pending = True
            return
        if self.sharded:
            u.grad_work = self.comm.reduce_scatter_sum(u.grads, u.grad_shard, async_op=True)
        else:
            u.grad_work = self.comm.all_reduce_sum(u.grads, async_op=True)

    _plane_pending = False

    # ---- exposed-communication meter ------------------------------------------------------------------
    # Time the COMPUTE stream spends waiting for communication: the join with the gradient reduce-scatter
    # stream after backward, and the barrier / scalar-exchange kernels of the optimizer phase.  Event pairs
    # are recorded only while `meter_comm` is on and are read (with a synchronise) by `exposed_comm_ms()`.
    meter_comm = False

    def _meter_begin(self):
        if not (self.meter_comm and self.device.type == "cuda"):
            return None
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def _meter_end(self, e0):
        if e0 is None:
            return
        e1 = torch.cuda.Event(enable_timing=True)
        e1.record()
        self._meter_pairs.append((e0, e1))

    def exposed_comm_ms(self, reset: bool = True) -> float:
        """Milliseconds the compute stream waited on communication since the last call."""
        if not self._meter_pairs:
            return 0.0
        torch.cuda.synchronize(self.device)
        total = sum(a.elapsed_time(b) for a, b in self._meter_pairs)
        if reset:
            self._meter_pairs = []
        return total

    def finish_grad_sync(self):
        e0 = self._meter_begin() if (self._plane_pending or any(u.grad_work is not None for u in self.units)) else None
        if self._plane_pending:
            plane = self.plane or self.ar_plane
            if self.ar_plane is not None:
                # all-reduce: peers store their slices into this rank's buffers; all of them have landed after a barrier
                with torch.cuda.stream(plane.stream):
                    plane.barrier()
            torch.cuda.current_stream().wait_stream(plane.stream)
            self._plane_pending = False
            self.reduce_seq += 1
        for u in self.units:
            if u.grad_work is not None:
                wait(u.grad_work)
                u.grad_work = None
        self._meter_end(e0)
        if self.average_on_sync and not self._averaged and self.world > 1 and not self.sharded and self.micro_step > 0:
            for u in self.units:
                u.grads.mul_(1.0 / self.world)
            self._averaged = True

    def grad_norm_and_clip(self, max_norm: float):
        """Global L2 norm of the (rank-averaged) gradient; leaves the clip coefficient on the device.
        Returns a 0-d tensor holding the norm."""
        self.finish_grad_sync()
        plane = self.plane or self.ar_plane
        if self.tp is not None:
            return self._grad_norm_and_clip_tp(max_norm, plane is not None)
        if plane is not None:
            # the reduce-scatter / all-reduce kernels already accumulated this rank's squared-norm partial
            e0 = self._meter_begin()
            # (the partials are of the rank-SUMMED gradient, also when the buffers have been averaged since)
            plane.global_clip_coef(self._sumsq, 1.0 / self.world, max_norm, self._clip)
            self._meter_end(e0)
            self.last_grad_norm = self._clip[1]
            return self._clip[1]
        self._sumsq.zero_()
        for u in self.units:
            O.sumsq_accumulate(u.grad_shard, self._sumsq)
        if self.sharded:
            e0 = self._meter_begin()
            self.comm.all_reduce_sum(self._sumsq)
            self._meter_end(e0)
        O.clip_coef(self._sumsq, 1.0 if self._averaged else 1.0 / self.world, max_norm, self._clip)
        self.last_grad_norm = self._clip[1]
        return self._clip[1]

    def _grad_norm_and_clip_tp(self, max_norm: float, have_partial: bool):
        """Tensor parallelism: the cut matrices count once per tp rank, the replicated parameters (the whole root unit
        and every block's vectors) once in all.  Two small sums: over this rank's data-parallel group, then over tp."""
        if not have_partial:
            self._sumsq.zero_()
            for u in self.units:
                O.sumsq_accumulate(u.grad_shard, self._sumsq)
        repl = torch.zeros(1, dtype=torch.float32, device=self.device)
        for u in self.units:
            lo, hi = u.shard_off, u.shard_off + u.shard_len
            a = lo if u is self.units[-1] else max(u.small_off, lo)
            b = min(u.layout.numel, hi)
            if a < b:
                O.sumsq_accumulate(u.grad_shard[a - lo:b - lo], repl)
        both = torch.cat([self._sumsq - repl, repl / self.tp.size])
        if self.sharded:
            self.comm.all_reduce_sum(both)
        self.tp.all_reduce_(both)
        total = both.sum().reshape(1)
        O.clip_coef(total, 1.0 if self._averaged else 1.0 / self.world, max_norm, self._clip)
        self.last_grad_norm = self._clip[1]
        return self._clip[1]

    def optimizer_step(self, opt: "EngineOptimizer"):
        """Fused update of every unit shard, then the gather of the new compute weights."""
        self.finish_grad_sync()
        if self.ecfg.grad_clip == 0.0 or opt.clip_pending is False:
            self._clip[0] = 1.0
        kind, use_clip = FUSED_OPTS[opt.opt_name]
        state_names = ["m", "v"] + (["tau"] if kind in _THREE_STATE else [])
        t = opt.step_count + 1
        g_decay, g_nodecay = opt.param_groups[0], opt.param_groups[1]
        diag = None
        if opt.want_diagnostics and kind not in (O.KIND_ADANA, O.KIND_DANA_STAR):
            # (the log-time family reports per-tensor metrics instead, recomputed from its state after the step)
            self._diag.zero_()
            diag = self._diag
        for u in self.units:
            u.ensure_state(state_names)
            lo, hi = u.shard_off, u.shard_off + u.shard_len
            for (a, b, grp) in ((0, u.layout.decay_end, g_decay), (u.layout.decay_end, u.layout.numel, g_nodecay)):
                s, e = max(a, lo), min(b, hi)
                if s >= e:
                    continue
                ls, le = s - lo, e - lo
                hyper = opt.hyper_for(grp, t)
                if self.plane is not None and u.weights is None:
                    # gathered weights: the new bf16 values of a flat range go to the ONE rank that owns those
                    # rows; ranges without a bf16 copy (norm weights, padding) only update their state
                    h = O.make_hyper(kind=kind, grad_scale=1.0 / self.world, **hyper)
                    tau = u.state.get("tau")

                    def step(a, b, dst=None, dst_off=0):
                        x0, x1 = a - lo, b - lo
                        tv = tau[x0:x1] if tau is not None else None
                        if dst is None:
                            O.fused_step(u.master[x0:x1], u.grad_shard[x0:x1], u.state["m"][x0:x1], u.state["v"][x0:x1],
                                         tv, None, kind=kind, grad_scale=1.0 / self.world, clip_coef_t=self._clip,
                                         diag=None, **hyper)
                        else:
                            self.plane.opt_step_push_to(u.master[x0:x1], u.grad_shard[x0:x1], u.state["m"][x0:x1],
                                                        u.state["v"][x0:x1], tv, [dst], dst_off, h, self._clip)

                    pos = s
                    for (flo, fhi, _owner, ptr) in u.segments:
                        a2, b2 = max(flo, s), min(fhi, e)
                        if a2 >= b2:
                            continue
                        if pos < a2:
                            step(pos, a2)
                        step(a2, b2, ptr, a2 - flo)
                        pos = b2
                    if pos < e:
                        step(pos, e)
                    continue
                if self.plane is not None:
                    h = O.make_hyper(kind=kind, grad_scale=1.0 / self.world, **hyper)
                    self.plane.opt_step_push(u.master[ls:le], u.grad_shard[ls:le], u.state["m"][ls:le],
                                             u.state["v"][ls:le], u.state["tau"][ls:le] if "tau" in u.state else None,
                                             u.weights, s, h, self._clip)
                    continue
                O.fused_step(u.master[ls:le], u.grad_shard[ls:le], u.state["m"][ls:le], u.state["v"][ls:le],
                             u.state["tau"][ls:le] if "tau" in u.state else None,
                             u.w_shard[ls:le] if u.low_precision else None,
                             kind=kind, grad_scale=1.0 / self.world, clip_coef_t=self._clip, diag=diag, **hyper)
            self._after_update(u)
        e0 = self._meter_begin()
        self._sync_small()     # (peer-memory plane: ends with the barrier that completes the weight pushes)
        self._meter_end(e0)
        if (self.plane or self.ar_plane) is not None:
            self._sumsq.zero_()
        opt.step_count = t
        self.opt_step_count += 1
        self.micro_step = 0
        if opt.want_diagnostics and kind in (O.KIND_ADANA, O.KIND_DANA_STAR):
            opt.diagnostics = self._per_tensor_optimizer_metrics(opt, kind, t)
        elif diag is not None:
            opt.absorb_diagnostics(diag, sum(u.layout.numel for u in self.units))

    @torch.no_grad()
    def _per_tensor_optimizer_metrics(self, opt, kind, t: int) -> Dict[str, float]:
        """The `optimizer/*` schedule metrics as the per-tensor optimizers define them (src/optim/dana_star_mk4.py:
        `current_alpha`, `auto_factor_mean`, `current_kappa_factor`, `m_norm` per parameter; src/optim/utils.py
        `log_optimizer_schedules` averages them over parameters).  They are functions of the state after the update, so
        they are recomputed from (m, v, tau) one parameter slot at a time on the iterations that log, and the fused step
        stays free of per-tensor reductions.  A sharded engine sums each slot's partial sums over the ranks."""
        expo = 1.0 - opt.kappa
        rows = []
        for u in self.units:
            lo, hi = u.shard_off, u.shard_off + u.shard_len
            for sl in u.layout.slots:
                a, b = max(sl.offset, lo), min(sl.offset + sl.numel, hi)
                if a >= b:
                    rows.append(torch.zeros(3, dtype=torch.float32, device=self.device))
                    continue
                grp = opt.param_groups[0] if sl.decay else opt.param_groups[1]
                eps = grp.get("epsilon", 1e-8)
                m, v = u.state["m"][a - lo:b - lo], u.state["v"][a - lo:b - lo]
                denom = torch.sqrt(v).add_(eps)
                if kind == O.KIND_ADANA:
                    mfac = m.abs().div_(denom)
                    af = mfac * float((1.0 + t) ** expo)
                else:
                    tau = u.state["tau"][a - lo:b - lo]
                    ct = tau.clamp(max=0.5)
                    floor = 1.0 / (1.0 + t)
                    reg = torch.relu(ct / (1.0 - ct) - floor).add_(floor)
                    mfac = m.abs().div_(denom).div_(torch.sqrt(reg))
                    af = (tau * t).clamp_(min=1.0).pow_(expo).mul_(mfac)
                if opt.clipsnr is not None:
                    af = af.clamp_(max=opt.clipsnr)
                rows.append(torch.stack([af.sum(dtype=torch.float64), mfac.sum(dtype=torch.float64),
                                         (m.double() ** 2).sum()]).float())
        table = torch.stack(rows)
        if self.sharded and self.world > 1:
            self.comm.all_reduce_sum(table)
        sums = table.double().cpu()
        n = torch.tensor([float(sl.numel) for u in self.units for sl in u.layout.slots], dtype=torch.float64)
        alpha, auto = sums[:, 0] / n, sums[:, 1] / n
        return {"current_alpha": float(alpha.mean()), "auto_factor_mean": float(auto.mean()),
                "current_kappa_factor": float((alpha / auto).mean()), "m_norm": float(sums[:, 2].sqrt().mean())}

    def _after_update(self, u: Unit):
        """Make the unit's compute weights current again after its shard was updated."""
        if self.plane is not None:
            return  # the optimizer kernel stored the new weights into every rank's buffer
        if self.world > 1 and self.sharded:
            u.gather_work = self.comm.all_gather(u.w_shard, u.weights, async_op=True)
        elif not u.low_precision and u.weights.data_ptr() != u.master.data_ptr():
            u.weights.copy_(u.master)

    def refresh_from_master(self):
        """Re-derive compute weights from the master copy (after an external optimizer or a load)."""
        with torch.no_grad():
            for u in self.units:
                if u.weights is None:            # gathered: every rank refills its own row slices
                    self._fill_slices(u, self._gather_full(u.master, u))
                    continue
                if self.plane is not None:
                    self.comm.all_gather(u.master.to(self.cdt), u.weights)
                    continue
                if u.low_precision or u.w_shard.data_ptr() != u.master.data_ptr():
                    u.w_shard.copy_(u.master)
                self._after_update(u)
            self._sync_small()

    def zero_grad(self):
        self.micro_step = 0
        if not self._grads_bound():
            self._bind_grads()

    def _grads_bound(self) -> bool:
        p = self._first_param
        return p is None or p.grad is not None

    def _bind_grads(self):
        """An optimizer that is not the engine's own may have dropped the parameters' `.grad` (`zero_grad(set_to_none=
        True)`): point them at the engine's gradient buffers again (replicated engines only: sharded ones expose none)."""
        params = dict(self.model.named_parameters())
        for u in self.units:
            if u.shard_len != u.padded:
                continue
            for s in u.layout.slots:
                params[s.name].grad = u.view(u.grads, s)

    # ---------------------------------------------------------------------------------------------
    # state dict (full tensors, reference key names) and sharded access
    # ---------------------------------------------------------------------------------------------
    def _gather_full(self, shard: torch.Tensor, u: Unit) -> torch.Tensor:
        if u.shard_len == u.padded:
            return shard
        full = torch.empty(u.padded, dtype=shard.dtype, device=shard.device)
        self.comm.all_gather(shard.contiguous(), full)
        return full

    def full_param_dict(self, which: str = "master") -> Dict[str, torch.Tensor]:
        """name -> full fp32 tensor (collective when sharded).  `which`: master | grad | m | v | tau.
        `grad` is the rank-summed gradient of the last synchronised backward, before averaging and clipping."""
        out = {}
        if which == "grad":
            self.finish_grad_sync()
        for u in self.units:
            src = u.master if which == "master" else u.grad_shard if which == "grad" else u.state.get(which)
            if src is None:
                continue
            full = self._gather_full(src, u)
            for s in u.layout.slots:
                out[s.name] = full[s.offset:s.offset + s.numel].view(s.shape).clone()
                if self.tp is not None:          # (collective over tp for the cut matrices)
                    out[s.name] = self.tp.gather_full(s.name, out[s.name])
                if self.tied and s.name == "transformer.wte.weight" and which == "master":
                    out["lm_head.weight"] = out[s.name]      # a state dict of tied modules names the tensor twice
        return out

    def load_full_param_dict(self, tensors: Dict[str, torch.Tensor], which: str = "master"):
        with torch.no_grad():
            for u in self.units:
                if which != "master":
                    u.ensure_state([which])
                dst = u.master if which == "master" else u.state[which]
                lo, hi = u.shard_off, u.shard_off + u.shard_len
                for s in u.layout.slots:
                    if s.name not in tensors:
                        continue
                    a, b = max(s.offset, lo), min(s.offset + s.numel, hi)
                    if a >= b:
                        continue
                    t = tensors[s.name]
                    if self.tp is not None and tuple(t.shape) != tuple(s.shape):
                        t = self.tp.local_part(s.name, t)           # a full tensor: keep this rank's heads / hidden units
                    src = t.reshape(-1)[a - s.offset:b - s.offset]
                    dst[a - lo:b - lo].copy_(src.to(dst.dtype))
        if which == "master":
            self.refresh_from_master()

    def state_dict(self):
        return self.full_param_dict("master")

    def num_params(self) -> int:
        return sum(s.numel for u in self.units for s in u.layout.slots)


class EngineOptimizer(torch.optim.Optimizer):
    """`torch.optim.Optimizer` facade over the engine's fused update.

    LR schedulers, `param_groups[i]['lr']`, `state_dict()` in the reference's layout
    (`state[idx] = {step, m, v[, tau]}`, groups `{lr, delta, epsilon, weight_decay,
    weighted_step_count, param_names}` with decay parameters first, each group sorted by
    name) all behave as with the per-tensor classes; the math runs in `Engine.optimizer_step`.
    """

    def __init__(self, engine: Engine, opt_name: str, args, group_specs):
        if opt_name not in FUSED_OPTS:
            raise ValueError(f"{opt_name} has no fused engine implementation")
        self.engine = engine
        self.opt_name = opt_name
        self.lr = args.lr
        self.kappa = getattr(args, "kappa", 1.0)
        self.clipsnr = getattr(args, "clipsnr", None) if FUSED_OPTS[opt_name][1] else None
        self.wd_decaying = getattr(args, "wd_decaying", False)
        self.wd_ts = getattr(args, "wd_ts", 1.0)
        self.gamma_3_factor = getattr(args, "gamma_3_factor", 1.0)
        self.betas = (getattr(args, "beta1", 0.9), getattr(args, "beta2", 0.95))
        self.step_count = 0
        self.clip_pending = None
        self.want_diagnostics = False
        self.diagnostics: Dict[str, float] = {}
        dev = engine.device
        groups = []
        for spec in group_specs:
            g = {"params": [nn.Parameter(torch.zeros(1, device=dev), requires_grad=False)],
                 "param_names": list(spec["param_names"] if "param_names" in spec else spec["params"])}
            if "weight_decay" in spec:
                g["weight_decay"] = spec["weight_decay"]
            groups.append(g)
        if opt_name.startswith("ademamix"):
            # the per-tensor classes' group keys (src/optim/ademamix.py:31-60), so schedulers and checkpoints agree
            defaults = dict(lr=args.lr, betas=(self.betas[0], self.betas[1], getattr(args, "adema_beta3", 0.9999)),
                            eps=1e-8, alpha=getattr(args, "adema_alpha", 2.0),
                            beta3_warmup=getattr(args, "adema_beta3_warmup", None),
                            alpha_warmup=getattr(args, "adema_alpha_warmup", None), weight_decay=args.weight_decay,
                            gamma_3_factor=self.gamma_3_factor)
            if opt_name == "ademamix-decaying-wd":
                defaults.update(wd_decaying=self.wd_decaying, wd_ts=self.wd_ts)
        elif opt_name.startswith("adamw"):
            defaults = dict(lr=args.lr, betas=self.betas, epsilon=1e-8, eps=1e-8, weight_decay=args.weight_decay)
        else:
            defaults = dict(lr=args.lr, delta=getattr(args, "delta", 8.0), epsilon=1e-8,
                            weight_decay=args.weight_decay, weighted_step_count=0)
        super().__init__(groups, defaults)

    def hyper_for(self, group, t: int) -> dict:
        lr = group["lr"]
        sched = lr / self.lr if self.lr != 0 else 0.0
        wd = group["weight_decay"]
        if self.opt_name == "adamw":
            wdf = 1.0 - lr * wd
        elif self.opt_name == "adamw-decaying-wd":
            wdf = wd_multiplier(wd, sched, t, self.wd_decaying, self.wd_ts) if wd != 0 else 1.0
        else:
            wdf = wd_multiplier(wd, sched, t, self.wd_decaying, self.wd_ts)
        if self.opt_name.startswith("ademamix"):
            from ..optim.adam_family import linear_hl_warmup_scheduler, linear_warmup_scheduler

            b1, b2, b3 = group["betas"]
            alpha = group["alpha"]
            if group.get("alpha_warmup") is not None:
                alpha = linear_warmup_scheduler(t, alpha_end=alpha, alpha_start=0, warmup=group["alpha_warmup"])
            if group.get("beta3_warmup") is not None:
                b3 = linear_hl_warmup_scheduler(t, beta_end=b3, beta_start=b1, warmup=group["beta3_warmup"])
            iwd = self.opt_name == "ademamix-decaying-wd"
            wdf = wd_multiplier(wd, sched, t, group.get("wd_decaying", False), group.get("wd_ts", 1.0)) if iwd else 1.0
            return dict(lr=lr, alpha=alpha, step=t, kappa=1.0, clipsnr=None, eps=group.get("eps", 1e-8),
                        gamma3=group.get("gamma_3_factor", 1.0), wd_factor=wdf, betas=(b1, b2), beta3=b3,
                        wd_coupled=0.0 if iwd else wd)
        delta = group.get("delta", 8.0)
        return dict(lr=lr, alpha=delta / (delta + t), step=t, kappa=self.kappa, clipsnr=self.clipsnr,
                    eps=group.get("epsilon", 1e-8), gamma3=self.gamma_3_factor, wd_factor=wdf, betas=self.betas)

    @torch.no_grad()
    def step(self, closure=None):
        for g in self.param_groups:
            if "weighted_step_count" in g:
                g["weighted_step_count"] += g["lr"] / self.lr if self.lr else 0.0
        self.engine.optimizer_step(self)
        self.clip_pending = None
        return None

    def zero_grad(self, set_to_none: bool = True):
        self.engine.zero_grad()

    def absorb_diagnostics(self, diag: torch.Tensor, numel: int):
        af, g2, mfac, m2 = (float(x) for x in diag.tolist())
        w = self.engine.world if self.engine.sharded else 1
        # sums over this rank's shard; a sharded engine reports rank-local means
        n = max(1, numel // w)
        self.diagnostics = {"current_alpha": af / n, "gradient_norm": math.sqrt(max(g2, 0.0)),
                            "auto_factor_mean": mfac / n, "m_norm": math.sqrt(max(m2, 0.0)),
                            "current_kappa_factor": (af / mfac) if mfac else 0.0}

    # ---- checkpoint format -----------------------------------------------------------------------
    def _ordered_names(self):
        return [n for g in self.param_groups for n in g["param_names"]]

    def state_dict(self):
        names = self._ordered_names()
        kind = FUSED_OPTS[self.opt_name][0]
        keys = {"m": "m", "v": "v", "tau": "tau"}
        if kind in (O.KIND_ADAMW, O.KIND_ADAMW_IWD):
            keys = {"m": "exp_avg", "v": "exp_avg_sq"}
        elif kind in (O.KIND_ADEMAMIX, O.KIND_ADEMAMIX_IWD):
            keys = {"m": "exp_avg_fast", "v": "exp_avg_sq", "tau": "exp_avg_slow"}
        fulls = {k: self.engine.full_param_dict(k) for k in keys}
        state = {}
        for i, n in enumerate(names):
            if not fulls["m"] or n not in fulls["m"]:
                continue
            st = {"step": self.step_count}
            for k, outk in keys.items():
                if fulls[k] and n in fulls[k]:
                    st[outk] = fulls[k][n]
            state[i] = st
        groups, off = [], 0
        for g in self.param_groups:
            gg = {k: v for k, v in g.items() if k != "params"}
            gg["params"] = list(range(off, off + len(g["param_names"])))
            off += len(g["param_names"])
            groups.append(gg)
        return {"state": state, "param_groups": groups}

    def load_state_dict(self, sd):
        names = self._ordered_names()
        kind = FUSED_OPTS[self.opt_name][0]
        keymap = {"m": "m", "v": "v", "tau": "tau"}
        if kind in (O.KIND_ADAMW, O.KIND_ADAMW_IWD):
            keymap = {"m": "exp_avg", "v": "exp_avg_sq"}
        elif kind in (O.KIND_ADEMAMIX, O.KIND_ADEMAMIX_IWD):
            keymap = {"m": "exp_avg_fast", "v": "exp_avg_sq", "tau": "exp_avg_slow"}
        state = sd.get("state", {})

        def plain(key):      # names as `torch.distributed.checkpoint` stores them, wrapper prefixes dropped
            while key.startswith(("_orig_mod.", "module.")):
                key = key.split(".", 1)[1]
            return key.replace("._orig_mod.", ".")

        by_name = {plain(k): v for k, v in state.items() if isinstance(k, str) and not k.isdigit()}
        for k, srck in keymap.items():
            tensors = {}
            for i, n in enumerate(names):
                # keyed by position (optimizer.state_dict()) or by parameter name (the reference's FSDP checkpoints)
                st = state.get(i, state.get(str(i), by_name.get(n)))
                if st is not None and srck in st:
                    tensors[n] = st[srck]
            if tensors:
                self.engine.load_full_param_dict(tensors, which=k)
        steps = [int(st["step"]) for st in state.values() if "step" in st]
        if steps:
            self.step_count = max(steps)
        for g, sg in zip(self.param_groups, sd.get("param_groups", [])):
            for k, v in sg.items():
                if k not in ("params",):
                    g[k] = v


def attach(model, cfg, comm: Optional[Comm] = None, sharded: bool = True, device=None,
           compute_dtype=None, tp_group=None) -> Engine:
    return Engine(model, cfg, comm=comm, sharded=sharded, device=device, compute_dtype=compute_dtype, tp_group=tp_group)
