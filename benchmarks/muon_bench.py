#!/usr/bin/env python
"""Distributed Muon's optimizer phase on one GPU: the Newton-Schulz chain per matrix shape, and a whole `d-muon` step of
a model's block stack through the kernel chain, through the torch-op path around the same GEMMs, and through the
per-tensor Muon class with library matmuls (what the reference runs per parameter, src/optim/muon.py:19-47, 519-567).

    python benchmarks/muon_bench.py [--model enoki36|qwen3] [--layers 4] [--iters 5]

One JSON line per measurement.  NS FLOPs per matrix: steps * (4 s^2 l + 2 s^3), s = short side, l = long side.
"""
import argparse
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))
from adana_b200.ops import _lib, muon_ns  # noqa: E402
from adana_b200.optim.muon import newton_schulz5  # noqa: E402

SHAPES = {"enoki36": [(6912, 2304), (2304, 2304), (9216, 2304), (2304, 9216)],
          "qwen3": [(2048, 2048), (1024, 2048), (6144, 2048), (2048, 6144)]}
MODEL = {"enoki36": dict(model="enoki", n_embd=2304, n_head=36, qkv_dim=64, mlp_hidden_dim=9216, sequence_length=2048),
         "qwen3": dict(model="qwen3", n_embd=2048, n_head=16, n_kv_head=8, qkv_dim=128, mlp_hidden_dim=6144,
                       sequence_length=4096, rope_theta=1e6)}


def timeit(fn, iters, flush=None):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    tot = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()                      # larger than L2: the next run starts cold
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        tot += e0.elapsed_time(e1)
    return tot / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="enoki36", choices=list(SHAPES))
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args()
    dev = "cuda:0"
    torch.manual_seed(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for shape in SHAPES[a.model]:
        s_, l_ = min(shape), max(shape)
        flops = 5 * (4.0 * s_ * s_ * l_ + 2.0 * s_ ** 3)
        G = torch.randn(*shape, device=dev).bfloat16()
        X = (G / (G.norm() + 1e-7)).contiguous()
        Y, A = torch.empty_like(X), torch.empty(s_, s_, dtype=torch.bfloat16, device=dev)
        B = torch.empty_like(A)
        work = X.clone()
        ours = timeit(lambda: muon_ns.ns_chain(work.copy_(X), Y, A, B, 5), a.iters, flush)
        lib_ms = timeit(lambda: newton_schulz5(G, 5), a.iters, flush)      # torch matmuls (cuBLAS) + elementwise passes
        print(json.dumps({"what": "newton_schulz5", "shape": shape, "ms": round(ours, 4), "tflops": round(flops / ours / 1e9, 1),
                          "torch_matmul_ms": round(lib_ms, 4), "speedup": round(lib_ms / ours, 3)}), flush=True)

    # ---- a whole optimizer step over `layers` blocks ------------------------------------------------------------
    from conftest import tiny_args
    from adana_b200.models.utils import get_model
    from adana_b200.optim.muon import Muon
    from adana_b200.parallel.dist_muon import ShardedMuon
    from adana_b200.runtime.engine import attach

    args = tiny_args(n_layer=a.layers, vocab_size=50304, opt="d-muon", lr=1e-3, weight_decay=0.1, momentum=0.95,
                     nesterov=True, muon_ns_steps=5, beta1=0.8, beta2=0.999, dtype="bfloat16", device=dev, grad_clip=1.0,
                     **MODEL[a.model])
    m = get_model(args).to(dev)
    eng = attach(m, args, device=dev, sharded=True)
    specs = m.get_parameter_group_specs()
    for g in specs:
        g["param_names"] = g["params"]
    opt = ShardedMuon(eng, args, specs)
    for u in eng.units:
        u.grad_shard.normal_(0, 1e-3)
    eng._clip[0] = 1.0
    opt.clip_pending = False

    def step():
        opt.step()

    n0 = _lib.launch_count()
    chain_ms = timeit(step, a.iters, flush)
    launches = (_lib.launch_count() - n0) // (a.iters + 3)
    saved, opt.chain = opt.chain, None
    torch_ms = timeit(step, a.iters, flush)
    opt.chain = saved
    # the per-tensor class on full tensors with torch matmuls: the reference's single-GPU Muon step
    params = [p for p in m.parameters()]
    full = [torch.nn.Parameter(p.detach().float().clone()) for p in params]
    mats = [p for p in full if p.dim() == 2 and p.shape[0] < 10000]
    rest = [p for p in full if not (p.dim() == 2 and p.shape[0] < 10000)]
    for p in full:
        p.grad = torch.randn_like(p) * 1e-3
    import adana_b200.optim.muon as MU

    ref = Muon(mats, lr=1e-3, momentum=0.95, nesterov=True, ns_steps=5, adamw_params=rest, adamw_lr=1e-3,
               adamw_betas=(0.8, 0.999), adamw_wd=0.1) if hasattr(MU, "Muon") else None
    per_tensor_ms = None
    if ref is not None:
        keep = MU.orthogonalize
        MU.orthogonalize = lambda G, steps: newton_schulz5(G, steps)       # library matmuls, as in the reference
        try:
            per_tensor_ms = timeit(lambda: ref.step(), a.iters, flush)
        except Exception as e:      # constructor / step signature differences must not hide the other numbers
            per_tensor_ms = f"unavailable: {type(e).__name__}: {e}"
        MU.orthogonalize = keep
    print(json.dumps({"what": f"d-muon optimizer step, {a.model} x {a.layers} blocks + root unit, 1 GPU",
                      "kernel_chain_ms": round(chain_ms, 3), "launches_per_step": launches,
                      "torch_ops_around_tcgen05_ns_ms": round(torch_ms, 3),
                      "per_tensor_class_torch_matmul_ms": per_tensor_ms if isinstance(per_tensor_ms, str) or per_tensor_ms is None
                      else round(per_tensor_ms, 3)}), flush=True)


if __name__ == "__main__":
    main()
