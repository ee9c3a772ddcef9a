"""`--opt` name -> optimizer object (24 names; reference: src/main.py:74-253).

On top of the reference's wiring, the names that have a fused flat-shard implementation
(`adana`, `dana-mk4`, `dana-star`, `dana-star-mk4`, `adamw`, `adamw-decaying-wd`) become an
`EngineOptimizer` whenever the kernel engine is attached to the model; every other name runs
its per-tensor class on the engine's parameter/gradient views (single / DDP) — `d-muon` under
the sharded engine goes through the distributed gather → Newton–Schulz → scatter chain.
"""
from __future__ import annotations

import inspect

import torch

from .adam_family import AdamWDecayingWD, AdEMAMix, AdEMAMixDecayingWD
from .logtime import ADana, DanaStarMK4
from .muon import DistributedMuon, Manau, Muon


def build_optimizer(args, model, group_specs, engine=None):
    """`group_specs`: [{"params": [tensors], "param_names": [...], ("weight_decay": 0.0)}, ...]."""
    from ..runtime.engine import FUSED_OPTS, EngineOptimizer

    if engine is not None and args.opt in FUSED_OPTS and not getattr(args, "no_fused_optimizer", False):
        return EngineOptimizer(engine, args.opt, args, group_specs)
    if engine is not None and getattr(engine, "tp", None) is not None:
        from .sharded_adapters import WHOLE_TENSOR

        if args.opt in WHOLE_TENSOR or args.opt == "d-muon":
            raise ValueError(f"--opt {args.opt} looks at whole matrices, which --tp_size > 1 cuts into per-rank parts on the "
                             f"kernel engine; use an element-wise optimizer or --tp_size 1")
    if engine is not None and args.opt == "d-muon" and (engine.sharded or engine.world == 1):
        # gather -> Newton-Schulz -> scatter on the engine's flat buffers (a kernel chain on a GPU), also on one rank
        from ..parallel.dist_muon import ShardedMuon

        return ShardedMuon(engine, args, group_specs)
    if engine is not None and engine.sharded:
        # every other name: its per-tensor class on views of this rank's shards (element-wise updates) or on whole
        # tensors kept by one owner rank each (updates that look at a matrix or a per-tensor norm)
        from .sharded_adapters import ELEMENTWISE, OwnerOptimizer, ShardViewOptimizer

        def make_inner(specs):
            return _build_per_tensor(args, model, specs)

        cls = ShardViewOptimizer if args.opt in ELEMENTWISE else OwnerOptimizer
        return cls(engine, make_inner, group_specs)
    if engine is not None:
        engine.average_on_sync = True      # a per-tensor class on the engine's gradient views wants rank-averaged gradients
    if engine is None and args.opt in ("muon", "soap", "adafactor") and \
            any(hasattr(p, "to_local") for g in group_specs for p in g["params"]):
        # a model without a kernel path under --distributed_backend fsdp: torch FSDP2 hands out DTensor shards.  These
        # three mix them with plain tensors (soap, adafactor) or partition the work by whole parameters per rank and
        # wait for each other (muon, the data-parallel form: src/optim/muon.py:443-602 needs `model.module`)
        raise ValueError(f"--opt {args.opt} does not run on parameters sharded by torch FSDP2 (this model has no kernel "
                         f"path); use --opt d-muon, --distributed_backend nccl, or a model configuration the engine takes")
    return _build_per_tensor(args, model, group_specs)


def _build_per_tensor(args, model, group_specs):
    """The per-tensor optimizer class of `args.opt` over the given parameter groups."""

    def adamw():
        cuda = "cuda" in str(args.device)
        fused = cuda and "fused" in inspect.signature(torch.optim.AdamW).parameters and getattr(args, "tp_size", 1) <= 1
        print(f"using fused AdamW: {fused}")
        return torch.optim.AdamW(group_specs, lr=args.lr, betas=(args.beta1, args.beta2),
                                 weight_decay=args.weight_decay, **({"fused": True} if fused else {}))

    def muon():
        raw = model.module if hasattr(model, "module") else model
        params = list(raw.parameters())
        if any(p.numel() == 0 for p in params):
            # sharded engine: the module's parameters are released; the groups hold the tensors this rank owns
            params = [p for g in group_specs for p in g["params"] if p.numel() > 0]
        return Muon(muon_params=params, lr=args.muon_lr_factor, momentum=args.momentum,
                    nesterov=args.nesterov, ns_steps=args.muon_ns_steps, adamw_params=None, adamw_lr=args.lr,
                    adamw_betas=(args.beta1, args.beta2), adamw_eps=1e-8, adamw_wd=args.weight_decay)

    def logtime(cls, clip):
        return lambda: cls(group_specs, lr=args.lr, delta=args.delta, kappa=args.kappa,
                           weight_decay=args.weight_decay, clipsnr=args.clipsnr if clip else None,
                           wd_decaying=args.wd_decaying, wd_ts=args.wd_ts, gamma_3_factor=args.gamma_3_factor)

    def ademamix(cls, extra):
        return lambda: cls(group_specs, lr=args.lr, betas=(args.beta1, args.beta2, args.adema_beta3),
                           alpha=args.adema_alpha, beta3_warmup=args.adema_beta3_warmup,
                           alpha_warmup=args.adema_alpha_warmup, weight_decay=args.weight_decay,
                           gamma_3_factor=args.gamma_3_factor, **extra)

    def zoo(name):
        from . import zoo as Z

        return Z.build(name, args, group_specs)

    registry = {
        "adamw": adamw,
        "sgd": lambda: torch.optim.SGD(group_specs, lr=args.lr, momentum=args.momentum,
                                       weight_decay=args.weight_decay, nesterov=args.nesterov),
        "muon": muon,
        "d-muon": lambda: DistributedMuon(group_specs, lr=args.lr, momentum=args.momentum, nesterov=args.nesterov,
                                          ns_steps=args.muon_ns_steps, adamw_betas=(args.beta1, args.beta2),
                                          adamw_eps=1e-8, weight_decay=args.weight_decay),
        "manau": lambda: Manau(group_specs, lr=args.lr, weight_decay=args.weight_decay,
                               matched_adamw_rms=getattr(args, "matched_adamw_rms", 0.2), momentum=args.momentum,
                               nesterov=args.nesterov, ns_steps=args.muon_ns_steps,
                               dana_momentum=getattr(args, "dana_momentum", False), delta=args.delta,
                               kappa=args.kappa, mk4A=args.mk4A, mk4B=args.mk4B, clipsnr=args.clipsnr, epsilon=1e-8,
                               weight_time=args.weight_time, wd_decaying=args.wd_decaying, wd_ts=args.wd_ts),
        "ademamix": ademamix(AdEMAMix, {}),
        "ademamix-decaying-wd": ademamix(AdEMAMixDecayingWD, dict(wd_decaying=args.wd_decaying, wd_ts=args.wd_ts)),
        "adana": logtime(ADana, False),
        "dana-mk4": logtime(ADana, True),
        "dana-star": logtime(DanaStarMK4, False),
        "dana-star-mk4": logtime(DanaStarMK4, True),
        "adamw-decaying-wd": lambda: AdamWDecayingWD(group_specs, lr=args.lr, betas=(args.beta1, args.beta2),
                                                     weight_decay=args.weight_decay, wd_decaying=args.wd_decaying,
                                                     wd_ts=args.wd_ts),
    }
    for name in ("soap", "lion", "sf-adamw", "sf-sgd", "signsgd", "signum", "prodigy", "sophiag", "adopt", "mars",
                 "adafactor", "lamb"):
        registry[name] = (lambda n=name: zoo(n))
    if args.opt not in registry:
        raise ValueError(f"Unknown optimizer: '{args.opt}'. Available: {sorted(registry)}")
    return registry[args.opt]()
