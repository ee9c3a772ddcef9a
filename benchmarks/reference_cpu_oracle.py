#!/usr/bin/env python
"""Loss-curve oracle: trains the small Enoki configuration on CPU with the UNMODIFIED reference classes and writes the
per-step losses (the source of `tests/golden/enoki3_cpu_reference_losses.json` and of the timed CPU baseline table).

    python benchmarks/reference_cpu_oracle.py --opt adana|dana-mk4|dana-star-mk4|adamw [--steps 200]
                                               [--ref_src baseline/_ref/src] [--out losses.json]

Recipe: enoki, 3 layers, 3 heads of 64, d 192, GELU MLP 768, vocabulary 50304, untied, fp32, batch 8 x 256; iid
Zipf(1.0) tokens (seed 0) read through the reference's DataReader(seed=1337); torch.manual_seed(0); lr 1e-3, warm-up
min(100, steps/2), cosine to ~0, gradient clip 0.5; kappa 0.85, delta 8, weight decay 4/wd_ts with wd_ts = steps/10
(AdamW: 4/(lr*steps), betas 0.9/0.999).  Shims: `tiktoken.get_encoding` is stubbed (no network access) and
TORCHDYNAMO_DISABLE=1 unless set otherwise (the reference compiles its optimizer updates; without a working host C++
toolchain for Inductor the flag runs the same math eagerly).
"""
import argparse
import json
import os
import sys
import time
import types
from pathlib import Path

import numpy as np

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
ROOT = Path(__file__).resolve().parent.parent


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--opt", default="adana", choices=["adana", "dana-mk4", "dana-star-mk4", "adamw"])
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--ref_src", default=str(ROOT / "baseline" / "_ref" / "src"))
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    if not (Path(a.ref_src) / "optim" / "adana.py").exists():
        sys.exit(f"no reference sources under {a.ref_src}")
    sys.path.insert(0, a.ref_src)
    import tiktoken

    tiktoken.get_encoding = lambda name: types.SimpleNamespace(name=name)
    import torch

    torch.manual_seed(0)
    import config as ref_config
    from data.utils import DataReader
    from models.utils import get_model
    from optim.schedule import cos_inf_schedule

    parser = argparse.ArgumentParser(allow_abbrev=False)
    parser.add_argument("--config_format", default="base")
    args = ref_config.parse_args_with_format(format="base", base_parser=parser, namespace=None, args=[
        "--model", "enoki", "--n_layer", "3", "--n_head", "3", "--n_embd", "192", "--qkv_dim", "64",
        "--mlp_hidden_dim", "768", "--sequence_length", "256", "--batch_size", "8", "--vocab_size", "50304",
        "--dtype", "float32", "--device", "cpu", "--weight_tying", "False", "--dropout", "0.0",
        "--init-scheme", "ScaledGPT", "--z_loss_coeff", "0.0"])
    vocab, steps = 50304, a.steps
    p = 1.0 / np.arange(1, vocab + 1, dtype=np.float64)
    p /= p.sum()
    tokens = np.random.default_rng(0).choice(vocab, size=8 * 257 * (steps + 64) + 4096, p=p).astype(np.uint16)
    reader = DataReader(tokens, local_batch_size=8, sequence_length=256, seed=1337, with_replacement=False,
                        auto_shard=False, keep_in_ram=True)
    reader.set_step(0)
    model = get_model(args)
    specs = model.get_parameter_group_specs()
    by_name = dict(model.named_parameters())
    for g in specs:
        g["params"] = [by_name[n] for n in g["params"]]
    lr, warm, wd_ts = 1e-3, min(100, steps // 2), max(steps // 10, 1)
    if a.opt == "adamw":
        opt = torch.optim.AdamW(specs, lr=lr, betas=(0.9, 0.999), weight_decay=4.0 / (lr * steps))
    else:
        kw = dict(lr=lr, delta=8.0, kappa=0.85, weight_decay=4.0 / wd_ts, wd_decaying=True, wd_ts=wd_ts, gamma_3_factor=1.0)
        if a.opt == "dana-star-mk4":
            from optim.dana_star_mk4 import DANA_STAR_MK4

            opt = DANA_STAR_MK4(specs, clipsnr=2.0, **kw)
        else:
            from optim.adana import ADana

            opt = ADana(specs, clipsnr=None if a.opt == "adana" else 2.0, **kw)
    sched = torch.optim.lr_scheduler.LambdaLR(opt, cos_inf_schedule(n_iterations=steps, n_warmup=warm, n_inf=0,
                                                                    div_factor=1e2, final_div_factor=1e8))
    losses, secs = [], []
    model.train()
    for it in range(steps):
        t0 = time.perf_counter()
        x, y = reader.sample_batch()
        out = model(x, targets=y)
        out["loss"].backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 0.5)
        opt.step()
        sched.step()
        opt.zero_grad(set_to_none=True)
        secs.append(time.perf_counter() - t0)
        losses.append(out["loss"].item())
        if it % 20 == 0 or it == steps - 1:
            print(f"it={it:4d} loss={losses[-1]:.4f} {secs[-1]:.3f} s", flush=True)
    med = float(np.median(secs[10:])) if steps > 10 else float(np.median(secs))
    res = {"opt": a.opt, "steps": steps, "zipf_entropy_nats": float(-(p * np.log(p)).sum()), "loss_mean_last10": float(np.mean(losses[-10:])),
           "sec_per_step_median": med, "tokens_per_sec": 8 * 256 / med, "losses": losses}
    if a.out:
        Path(a.out).write_text(json.dumps(res))
    print(json.dumps({k: v for k, v in res.items() if k != "losses"}))


if __name__ == "__main__":
    main()
