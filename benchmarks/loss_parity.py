#!/usr/bin/env python
"""Loss-curve parity on a GPU: the same small Enoki model, the same initial weights (`--init_compat reference`), the
same token batches and the same optimizer settings, trained once with this framework (kernel engine, bf16 compute,
fp32 master weights, fused Dana-Star-MK4) and once with the reference's own model / optimizer classes (bf16 autocast).

    python benchmarks/loss_parity.py --arm ours      --steps 1000 --out out/parity_ours.json
    python benchmarks/loss_parity.py --arm reference --steps 1000 --out out/parity_ref.json
    python benchmarks/loss_parity.py --compare out/parity_ours.json out/parity_ref.json

`--dtype float32 --size enoki12` is the fp32 comparison at the 12-layer size (TF32 off on both arms).

The reference arm imports the unmodified reference from baseline/_ref/src (tiktoken stubbed: no network).
"""
import argparse
import json
import sys
import time
import types
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent

MODEL_ARGS = ["--model", "enoki", "--n_layer", "6", "--n_head", "6", "--n_embd", "384", "--qkv_dim", "64",
              "--mlp_hidden_dim", "1536", "--sequence_length", "512", "--batch_size", "16", "--vocab_size", "50304",
              "--weight_tying", "False", "--dropout", "0.0", "--init-scheme", "ScaledGPT", "--z_loss_coeff", "0.0"]
SIZES = {"small": dict(n_layer=6, n_head=6, n_embd=384, mlp_hidden_dim=1536),
         "enoki12": dict(n_layer=12, n_head=12, n_embd=768, mlp_hidden_dim=3072)}
LR, KAPPA, DELTA, CLIPSNR, GRAD_CLIP = 1e-3, 0.85, 8.0, 2.0, 0.5


def model_args(size):
    out = list(MODEL_ARGS)
    for k, v in SIZES[size].items():
        out[out.index("--" + k) + 1] = str(v)
    return out


def tokens(steps):
    V = 50304
    rng = np.random.default_rng(0)
    p = 1.0 / np.arange(1, V + 1, dtype=np.float64)
    p /= p.sum()
    return rng.choice(V, size=16 * 513 * (steps + 8) + 4096, p=p).astype(np.uint16)


def run(arm, steps, dtype, size="small"):
    import argparse as ap

    MODEL_ARGS = model_args(size)
    # fp32 runs use plain fp32 multiplies on both arms (no TF32)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False

    warm, wd_ts = max(1, steps // 10), max(1, steps // 10)
    wd = 4.0 / wd_ts
    parser = ap.ArgumentParser(allow_abbrev=False)
    parser.add_argument("--config_format", default="base")
    torch.manual_seed(0)
    if arm == "reference":
        sys.path.insert(0, str(ROOT / "baseline" / "_ref" / "src"))
        import tiktoken

        tiktoken.get_encoding = lambda name: types.SimpleNamespace(name=name)
        import config as rcfg
        from data.utils import DataReader
        from models.utils import get_model
        from optim.dana_star_mk4 import DANA_STAR_MK4
        from optim.schedule import cos_inf_schedule

        args = rcfg.parse_args_with_format(format="base", base_parser=parser, namespace=None,
                                           args=MODEL_ARGS + ["--dtype", dtype, "--device", "cuda:0"])
        model = get_model(args).to("cuda")
        specs = model.get_parameter_group_specs()
        named = dict(model.named_parameters())
        for g in specs:
            g["params"] = [named[n] for n in g["params"]]
        opt = DANA_STAR_MK4(specs, lr=LR, delta=DELTA, kappa=KAPPA, weight_decay=wd, clipsnr=CLIPSNR, wd_decaying=True,
                            wd_ts=wd_ts, gamma_3_factor=1.0)
        lam = cos_inf_schedule(n_iterations=steps, n_warmup=warm, n_inf=0, div_factor=1e2, final_div_factor=1e8)
        ctx = torch.amp.autocast("cuda", dtype=torch.bfloat16) if dtype == "bfloat16" else torch.amp.autocast("cuda", enabled=False)
        clip = lambda: torch.nn.utils.clip_grad_norm_(model.parameters(), GRAD_CLIP)
    else:
        sys.path.insert(0, str(ROOT))
        from adana_b200.config import parse_args_with_format
        from adana_b200.data.readers import DataReader
        from adana_b200.models.utils import get_model
        from adana_b200.optim.schedule import CosInf
        from adana_b200.runtime.engine import EngineOptimizer, attach

        args = parse_args_with_format(format="base", base_parser=parser, namespace=None,
                                      args=MODEL_ARGS + ["--dtype", dtype, "--device", "cuda:0", "--init_compat", "reference",
                                                         "--grad_clip", str(GRAD_CLIP)])
        for k, v in dict(opt="dana-star-mk4", lr=LR, delta=DELTA, kappa=KAPPA, weight_decay=wd, clipsnr=CLIPSNR,
                         wd_decaying=True, wd_ts=wd_ts, gamma_3_factor=1.0, acc_steps=1).items():
            setattr(args, k, v)
        model = get_model(args).to("cuda")
        eng = attach(model, args, device="cuda:0")
        specs = model.get_parameter_group_specs()
        for g in specs:
            g["param_names"] = g["params"]
        opt = EngineOptimizer(eng, "dana-star-mk4", args, specs)
        lam = CosInf(steps, warm, 1e2, 1e8, 0)
        ctx = torch.amp.autocast("cuda", enabled=False)
        clip = lambda: eng.grad_norm_and_clip(GRAD_CLIP)
    reader = DataReader(tokens(steps), 16, 512, seed=1337, with_replacement=False, auto_shard=False, keep_in_ram=True)
    reader.set_step(0)
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lam)
    model.train()
    losses = []
    t0 = time.time()
    for _ in range(steps):
        x, y = reader.sample_batch()
        x, y = x.cuda(), y.cuda()
        with ctx:
            out = model(x, targets=y)
        out["loss"].backward()
        clip()
        opt.step()
        sched.step()
        opt.zero_grad(set_to_none=True)
        losses.append(out["loss"].detach())
    torch.cuda.synchronize()
    return {"arm": arm, "dtype": dtype, "size": size, "steps": steps, "seconds": time.time() - t0,
            "losses": [float(v) for v in torch.stack(losses).float().cpu()]}


def compare(a_path, b_path, window=20):
    a, b = (json.loads(Path(p).read_text()) for p in (a_path, b_path))
    la, lb = np.array(a["losses"]), np.array(b["losses"])
    n = min(len(la), len(lb))
    la, lb = la[:n], lb[:n]
    rel = np.abs(la - lb) / lb
    k = np.ones(window) / window
    sa, sb = np.convolve(la, k, mode="valid"), np.convolve(lb, k, mode="valid")
    srel = np.abs(sa - sb) / sb
    rep = {"a": a["arm"], "b": b["arm"], "steps": n, "first_loss": [float(la[0]), float(lb[0])],
           "dtype": [a.get("dtype"), b.get("dtype")], "size": [a.get("size"), b.get("size")],
           "within_1pct_pointwise": bool(rel.max() < 0.01), "within_1pct_smoothed": bool(srel.max() < 0.01),
           "final_mean_last50": [float(la[-50:].mean()), float(lb[-50:].mean())],
           "per_step_rel_diff": {"first10_max": float(rel[:10].max()), "median": float(np.median(rel)),
                                 "p95": float(np.quantile(rel, 0.95)), "max": float(rel.max())},
           f"smoothed{window}_rel_diff": {"median": float(np.median(srel)), "p95": float(np.quantile(srel, 0.95)),
                                          "max": float(srel.max())},
           "every_100": [[int(i), float(la[i]), float(lb[i])] for i in range(0, n, max(1, n // 10))]}
    print(json.dumps(rep, indent=1))


if __name__ == "__main__":
    ap_ = argparse.ArgumentParser()
    ap_.add_argument("--arm", choices=["ours", "reference"])
    ap_.add_argument("--steps", type=int, default=1000)
    ap_.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap_.add_argument("--size", default="small", choices=sorted(SIZES), help="enoki12: 12 layers, d 768 (124 M parameters)")
    ap_.add_argument("--out", default=None)
    ap_.add_argument("--compare", nargs=2)
    a = ap_.parse_args()
    if a.compare:
        compare(*a.compare)
    else:
        res = run(a.arm, a.steps, a.dtype, a.size)
        print(json.dumps({k: v for k, v in res.items() if k != "losses"} | {"loss_first": res["losses"][0], "loss_last": res["losses"][-1]}))
        if a.out:
            Path(a.out).parent.mkdir(parents=True, exist_ok=True)
            Path(a.out).write_text(json.dumps(res))
