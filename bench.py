#!/usr/bin/env python
"""Headline benchmark: whole-job training tokens/s of Enoki-36 (36 layers, d 2304, ~2.5 B
parameters) with dana-star-mk4 under the fsdp backend, bf16 compute / fp32 state, on N GPUs of
one node, synthetic Zipf(1.0) tokens, random-init weights.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Weak scaling: every GPU processes 64 sequences of 2048 tokens per optimizer step (8 micro-steps
of 8 sequences), i.e. global batch 64*N (512 at N = 8).  One JSON line is printed by rank 0.

Two measurements of the same metric:
  value  device-timed: K optimizer steps bracketed by barrier + synchronize, CUDA events, max
         over ranks; the step's token batches already sit on the device.
  e2e    the same K steps driven through the public training API (`Trainer.train_step`): every
         micro-batch is gathered from the token file into pinned host memory, copied to the
         device, and the step's loss is read back to the host.

`--impl reference` runs the unmodified reference (baseline/_ref/src) through its own `main()` /
`train()` on the same model, optimizer, batch and data shape and prints the same line with
"impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# Benchmark configurations.  `enoki36` is the headline (the only one the default command line runs); the others are
# the remaining training configurations of the benchmark list: the 12-layer Enoki at 32 sequences per GPU (global
# batch 256 on 8 GPUs), and the Qwen3-style decoder (28 layers, 16 query / 8 KV heads of 128, SwiGLU 6144, RoPE
# theta 1e6, sequence 4096) trained with distributed Muon.
CONFIGS = {
    "enoki36": dict(
        label="enoki-36 (L{n_layer}, d2304, mlp9216, hd64, V50304)", metric_model="enoki-36",
        model=dict(model="enoki", n_layer=36, n_head=36, n_embd=2304, qkv_dim=64, mlp_hidden_dim=9216,
                   sequence_length=2048, vocab_size=50304),
        per_gpu_seqs=64, micro_batch=8, opt="dana-star-mk4"),
    "enoki12": dict(
        label="enoki-12 (L{n_layer}, d768, mlp3072, hd64, V50304)", metric_model="enoki-12",
        model=dict(model="enoki", n_layer=12, n_head=12, n_embd=768, qkv_dim=64, mlp_hidden_dim=3072,
                   sequence_length=2048, vocab_size=50304),
        per_gpu_seqs=32, micro_batch=16, opt="dana-star-mk4"),
    "qwen3-muon": dict(
        label="qwen3 (L{n_layer}, d2048, 16Q/8KV x hd128, swiglu 6144, theta 1e6, V50304)", metric_model="qwen3-1.7B",
        model=dict(model="qwen3", n_layer=28, n_head=16, n_kv_head=8, n_embd=2048, qkv_dim=128, mlp_hidden_dim=6144,
                   sequence_length=4096, vocab_size=50304, rope_theta=1e6, elementwise_attn_output_gate=False,
                   normalization_layer_type="rmsnorm"),
        per_gpu_seqs=32, micro_batch=4, opt="d-muon"),
}
OPTS = {
    "dana-star-mk4": dict(opt="dana-star-mk4", kappa=0.85, delta=8.0, clipsnr=2.0, lr=4.6e-5, weight_decay=4.0 / 100.0,
                          wd_ts=100.0, wd_decaying=True, grad_clip=0.5, z_loss_coeff=1e-4),
    "dana-mk4": dict(opt="dana-mk4", kappa=0.85, delta=8.0, clipsnr=2.0, lr=4.6e-5, weight_decay=4.0 / 100.0,
                     wd_ts=100.0, wd_decaying=True, grad_clip=0.5, z_loss_coeff=1e-4),
    "adamw": dict(opt="adamw", beta1=0.9, beta2=0.95, lr=3e-4, weight_decay=0.1, grad_clip=0.5, z_loss_coeff=1e-4),
    "d-muon": dict(opt="d-muon", lr=1e-3, momentum=0.95, nesterov=True, muon_ns_steps=5, beta1=0.8, beta2=0.999,
                   weight_decay=0.01, grad_clip=0.5, z_loss_coeff=1e-4),
}
MODEL = CONFIGS["enoki36"]["model"]


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=5)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--config", default="enoki36", choices=sorted(CONFIGS))
    p.add_argument("--opt", default=None, choices=sorted(OPTS), help="default: the configuration's own optimizer")
    p.add_argument("--micro_batch", type=int, default=None)
    p.add_argument("--per_gpu_seqs", type=int, default=None)
    p.add_argument("--n_layer", type=int, default=None, help="override for smoke runs only")
    p.add_argument("--tp_size", type=int, default=1, help="tensor-parallel ranks per data-parallel replica (both arms)")
    p.add_argument("--no_e2e", action="store_true")
    p.add_argument("--attention", default="auto", choices=["auto", "native", "sdpa"])
    p.add_argument("--ref_no_compile", action="store_true")
    p.add_argument("--fsdp_weights", default="resident", choices=["resident", "gathered"],
                   help="ours: keep the bf16 block matrices resident on every rank, or as row slices fetched by the GEMMs")
    a = p.parse_args()
    c = CONFIGS[a.config]
    a.micro_batch = a.micro_batch or c["micro_batch"]
    a.per_gpu_seqs = a.per_gpu_seqs or c["per_gpu_seqs"]
    a.n_layer = a.n_layer or c["model"]["n_layer"]
    a.opt = a.opt or c["opt"]
    return a


def shared_config(a, world: int) -> dict:
    """The keys that name the workload; identical for both arms (implementation choices go to `impl_detail`)."""
    c = CONFIGS[a.config]
    dp = world // a.tp_size
    return {"model": c["label"].format(n_layer=a.n_layer), "global_batch": a.per_gpu_seqs * dp,
            "seq_len": c["model"]["sequence_length"], "micro_batch": a.micro_batch,
            "acc_steps": a.per_gpu_seqs // a.micro_batch, "optimizer": a.opt,
            "parallelism": f"fsdp{dp}" + (f"xtp{a.tp_size}" if a.tp_size > 1 else "")}


def metric_name(a) -> str:
    return f"tokens/sec/box FSDP {a.opt} {CONFIGS[a.config]['metric_model']}"


def dist_env(gpus: int):
    """Single-GPU runs are started without torchrun: provide the rendezvous variables."""
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(29500 + os.getpid() % 2000))
    return int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])


def write_tokens(n_tokens: int, seed: int = 0) -> Path:
    """Synthetic Zipf(1.0) corpus in the fineweb-10BT layout (train.bin / val.bin, uint16)."""
    from adana_b200.data.datasets import make_zipf_tokens

    root = Path(os.environ.get("ADANA_BENCH_DATA", "/tmp/adana_bench_data")) / "fineweb-10BT"
    root.mkdir(parents=True, exist_ok=True)
    tr, va = root / "train.bin", root / "val.bin"
    if not tr.exists() or tr.stat().st_size != 2 * n_tokens:
        tmp = root / f"train.{os.getpid()}.tmp"
        make_zipf_tokens(n_tokens, 50304, 1.0, seed).tofile(tmp)
        os.replace(tmp, tr)
    if not va.exists():
        tmp = root / f"val.{os.getpid()}.tmp"
        make_zipf_tokens(300_000, 50304, 1.0, seed + 1).tofile(tmp)
        os.replace(tmp, va)
    return root.parent


def _attention_impl() -> str:
    from adana_b200.ops import attention as att

    mode = att.get_mode()
    native = mode == "native" or (mode == "auto" and att._lib.available() and att._lib.has("adana_attn_bwd"))
    return "tcgen05 kernels (csrc/attention_tcgen05.cu)" if native else "torch SDPA (cuDNN library kernel)"


def emit(payload: dict):
    print(json.dumps(payload), flush=True)


# =================================================================================================
# our implementation
# =================================================================================================
def run_ours(a):
    import torch
    import torch.distributed as dist

    from adana_b200 import distributed
    from adana_b200.config import flags
    from adana_b200.data import DataReader
    from adana_b200.models.utils import get_model
    from adana_b200.ops import _lib
    from adana_b200.optim.registry import build_optimizer
    from adana_b200.optim.schedule import build_scheduler
    from adana_b200.main import named_param_groups
    from adana_b200.train.loop import Trainer
    from adana_b200.utils.timing import ClockSampler

    rank, local_rank, world = dist_env(a.gpus)
    assert world == a.gpus, f"--gpus {a.gpus} but WORLD_SIZE={world}"
    acc = a.per_gpu_seqs // a.micro_batch
    args = flags.defaults()
    conf = CONFIGS[a.config]
    for k, v in {**conf["model"], **OPTS[a.opt]}.items():
        setattr(args, k, v)
    args.n_layer = a.n_layer
    args.dtype, args.device = "bfloat16", f"cuda:{local_rank}"
    args.distributed_backend = "fsdp"
    # the backend's split rule (acc //= gcd(acc, N); batch //= N / gcd) maps this to
    # micro-batch `micro_batch` and `acc` accumulation steps on every rank
    dp = world // a.tp_size
    args.tp_size = a.tp_size
    args.batch_size, args.acc_steps = a.micro_batch, acc * dp
    args.weight_tying, args.init_scheme = False, "ScaledGPT"
    # (the same schedule flags as the reference arm: the two arms' learning rates, and so their losses, are comparable)
    args.scheduler, args.iterations, args.warmup_steps = "cos_inf", a.warmup + a.steps, 1
    args.final_div_factor, args.dataset, args.log_interval = 0.1, "fineweb", 0
    args.attention = a.attention
    args.fsdp_weights = a.fsdp_weights
    steps_total = a.warmup + a.steps
    tokens_needed = (2 * steps_total + 4) * a.per_gpu_seqs * world * (conf["model"]["sequence_length"] + 1) + 4_000_000
    if rank == 0:
        args.datasets_dir = str(write_tokens(tokens_needed))
    torch.cuda.set_device(local_rank)
    backend = distributed.make_backend_from_args(args)
    backend.comm.barrier()
    args.datasets_dir = str(Path(os.environ.get("ADANA_BENCH_DATA", "/tmp/adana_bench_data")))
    args = backend.get_adjusted_args_for_process(args)
    assert (args.batch_size, args.acc_steps) == (a.micro_batch, acc)
    torch.manual_seed(0)
    with torch.device(args.device):   # initialise on the GPU: seconds instead of minutes for 2.5 B parameters
        model = get_model(args)
    model = backend.transform_model(model)
    specs, _ = named_param_groups(model, backend)
    opt = build_optimizer(args, model, specs, engine=backend.engine)
    backend.engine_optimizer = hasattr(opt, "engine")
    sched = build_scheduler(args, opt)
    train_reader = DataReader(Path(args.datasets_dir) / "fineweb-10BT" / "train.bin", args.batch_size,
                              args.sequence_length, seed=1337, auto_shard=True, keep_in_ram=True)
    val_reader = DataReader(Path(args.datasets_dir) / "fineweb-10BT" / "val.bin", args.batch_size,
                            args.sequence_length, seed=1337, auto_shard=False, keep_in_ram=True)
    trainer = Trainer(model, opt, {"train": train_reader, "val": val_reader}, sched, "/tmp/adana_bench_exp",
                      backend, args)
    model.train()
    tokens_per_step = a.per_gpu_seqs * dp * args.sequence_length

    # ---- device-timed region: batches pre-staged on the device ---------------------------------------
    dev_batches = []
    for _ in range(acc * 2):
        x, y = train_reader.sample_batch()
        dev_batches.append((x.to(args.device), y.to(args.device)))

    if getattr(backend, "engine", None) is not None:
        backend.engine.report_aux = False      # nothing logs in the timed steps (log_interval 0), as in Trainer.train_step
    phase_marks = []       # per timed step: events after (last backward launched, clip, optimizer step)

    def step_device(i, mark=False):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if mark else None
        if mark:
            ev[0].record()
        for m in range(acc):
            x, y = dev_batches[(i * acc + m) % len(dev_batches)]
            with backend.get_context_for_microstep_forward(model, m, acc):
                out = model(x, targets=y)
            (out["loss"] / acc).backward()
        if mark:
            ev[1].record()
        backend.clip_grad_norm_(None, args.grad_clip)
        if mark:
            ev[2].record()
        opt.step()
        sched.step()
        opt.zero_grad()
        if mark:
            ev[3].record()
            phase_marks.append(ev)

    for i in range(a.warmup):
        step_device(i)
    torch.cuda.synchronize()
    backend.comm.barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _lib.launch_count()
    engine = getattr(backend, "engine", None)
    if engine is not None and world > 1:
        engine.meter_comm = True       # event pairs around every point where the compute stream waits on communication
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for i in range(a.steps):
        step_device(a.warmup + i, mark=True)
    e1.record()
    torch.cuda.synchronize()
    backend.comm.barrier()
    clocks = sampler.stop() if rank == 0 else None
    launches = _lib.launch_count() - launches0
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=args.device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms.item()) / a.steps
    exposed = None
    if engine is not None and world > 1:
        ex = torch.tensor([engine.exposed_comm_ms()], dtype=torch.float64, device=args.device)
        engine.meter_comm = False
        dist.all_reduce(ex, op=dist.ReduceOp.MAX)
        exposed = {"ms_per_step": float(ex.item()) / a.steps, "fraction_of_step": float(ex.item()) / a.steps / ms_per_step,
                   "what": "time the compute stream waited on gradient reduce-scatter joins, barriers and scalar exchanges (max over ranks)"}
    _lib.check_status()
    # where the step goes, on the device: forward+backward of all micro-steps (gradient reduce-scatters of finished
    # units overlap it), the join with the reduce-scatter stream + gradient norm + clip coefficient, and the optimizer
    # step with the push of the new weights.  `skew` is max - min over ranks of the forward+backward time: what a
    # rank spends waiting for the slowest one at the next barrier.
    ph = torch.tensor([[ev[k].elapsed_time(ev[k + 1]) for k in range(3)] for ev in phase_marks],
                      dtype=torch.float64, device=args.device).mean(0)
    ph_max, ph_min = ph.clone(), ph.clone()
    if world > 1:
        dist.all_reduce(ph_max, op=dist.ReduceOp.MAX)
        dist.all_reduce(ph_min, op=dist.ReduceOp.MIN)
    phases = {"fwd_bwd_ms": float(ph_max[0]), "grad_sync_tail_and_clip_ms": float(ph_max[1]),
              "optimizer_and_weight_push_ms": float(ph_max[2]), "fwd_bwd_skew_ms": float(ph_max[0] - ph_min[0]),
              "what": "device time per optimizer step, max over ranks (skew: max - min over ranks)"}

    # ---- end-to-end region: public API, pinned host batches, loss read back every step ----------------
    e2e = None
    if not a.no_e2e:
        trainer.stager.lookahead = True
        for _ in range(1):
            out, loss = trainer.train_step()
            float(loss.item())
        torch.cuda.synchronize()
        backend.comm.barrier()
        t0 = time.perf_counter()
        for _ in range(a.steps):
            out, loss = trainer.train_step()
            float(loss.item())      # device -> host read of the step's result
        torch.cuda.synchronize()
        dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=args.device)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        e2e = {"value": tokens_per_step * a.steps / float(dt.item()), "unit": "tokens/s",
               "h2d_bytes_per_step": int(trainer.stager.bytes_per_batch * acc), "d2h_bytes_per_step": 4,
               "ms_per_step": 1e3 * float(dt.item()) / a.steps}
        _lib.check_status()
    final_loss = float(out["loss"].item()) if not a.no_e2e else None
    mem = torch.cuda.max_memory_allocated() / 2 ** 30
    if rank == 0:
        emit({"metric": metric_name(a), "value": tokens_per_step / (ms_per_step / 1e3),
              "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms_per_step,
              "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
              "data": "synthetic Zipf(1.0) tokens, random-init weights", "impl": "ours",
              "config": shared_config(a, world),
              "impl_detail": {"l2": "inputs and weights exceed the 126 MB L2", "attention": _attention_impl(),
                              "fsdp_weights": a.fsdp_weights,
                              "fsdp_comm": "peer-memory kernels" if getattr(engine, "plane", None) is not None
                              else ("nccl" if world > 1 else "none (one GPU)"),
                              "reduce_dtype": getattr(getattr(engine, "ecfg", None), "reduce_dtype", None)},
              "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "exposed_comm": exposed, "phases": phases,
              "peak_mem_gib": round(mem, 2), "final_loss": final_loss})
    backend.finalize()


# =================================================================================================
# reference implementation (unmodified sources under baseline/_ref)
# =================================================================================================
def run_reference(a):
    ref_src = ROOT / "baseline" / "_ref" / "src"
    if not (ref_src / "main.py").exists():
        emit({"impl": "reference", "unavailable": "baseline/_ref/src is missing (reference not installed)"})
        return
    rank, local_rank, world = dist_env(a.gpus)
    # a rank that fails or never joins would leave the others waiting in their first collective: a failing
    # rank leaves a note that every rank's watchdog thread polls, and the whole arm has a time limit
    import threading

    limit = float(os.environ.get("ADANA_REF_TIMEOUT", "900"))
    note = Path(os.environ.get("ADANA_BENCH_DATA", "/tmp/adana_bench_data")) / f"ref_failed.{os.environ.get('MASTER_PORT', '0')}"
    note.parent.mkdir(parents=True, exist_ok=True)
    if rank == 0 and note.exists():
        note.unlink()
    done = threading.Event()

    def watch():
        t_start = time.time()
        while not done.wait(2.0):
            why = None
            if note.exists():
                why = "a rank failed: " + note.read_text()[:300]
            elif time.time() - t_start > limit:
                why = f"the reference did not finish within {limit:.0f} s on {world} GPU(s)"
            if why:
                if rank == 0:
                    emit({"impl": "reference", "unavailable": why})
                os._exit(0)

    threading.Thread(target=watch, daemon=True).start()
    try:
        import torch
        import torch.distributed as dist

        # launcher-side accommodations (no reference file is touched): the GPT-2 BPE files cannot be
        # downloaded here, and the reference creates a tokenizer object in every model constructor
        import tiktoken

        class _NoTokenizer:
            eot_token = 50256

            def encode(self, *_, **__):
                return [0]

            encode_ordinary = encode

            def decode(self, *_):
                return ""

        tiktoken.get_encoding = lambda name: _NoTokenizer()
        sys.path.insert(0, str(ref_src))
        os.chdir(ref_src)
        import main as ref_main  # the reference's entry module

        acc = a.per_gpu_seqs // a.micro_batch
        steps_total = a.warmup + a.steps
        seq_len = CONFIGS[a.config]["model"]["sequence_length"]
        tokens_needed = (2 * steps_total + 4) * a.per_gpu_seqs * world * (seq_len + 1) + 4_000_000
        data_root = Path(os.environ.get("ADANA_BENCH_DATA", "/tmp/adana_bench_data"))
        # rank 0 writes the corpus; the others must not reach the reference's dataset code (which would try
        # to download a missing corpus) before the files exist, and no process group is up yet to wait on
        marker = data_root / f"ready.{tokens_needed}.{os.environ.get('MASTER_PORT', '0')}"
        if rank == 0:
            write_tokens(tokens_needed)
            marker.write_text("ok")
        else:
            t_wait = time.time()
            while not marker.exists():
                if time.time() - t_wait > 600:
                    raise RuntimeError("rank 0 did not finish writing the synthetic corpus within 600 s")
                time.sleep(0.5)
        conf = CONFIGS[a.config]
        md = conf["model"]
        if md["model"] == "qwen3" and md.get("n_kv_head", md["n_head"]) != md["n_head"]:
            # the reference's Qwen3 has neither grouped-query attention nor a RoPE-theta flag
            # (src/models/qwen3.py:116-133, src/config/base.py:266-348): this configuration cannot be stated on its CLI
            emit({"impl": "reference", "unavailable": "the reference's qwen3 model has no GQA (n_kv_head) and no "
                  "rope_theta option; config qwen3-muon cannot be expressed on its command line"})
            done.set()
            return
        argv = ["--model", md["model"], "--n_layer", str(a.n_layer), "--n_head", str(md["n_head"]),
                "--n_embd", str(md["n_embd"]), "--qkv_dim", str(md["qkv_dim"]), "--mlp_hidden_dim",
                str(md["mlp_hidden_dim"]), "--sequence_length", str(md["sequence_length"]), "--vocab_size", "50304",
                "--weight_tying", "False", "--init-scheme", "ScaledGPT", "--dtype", "bfloat16",
                "--distributed_backend", "fsdp", "--device", f"cuda:{local_rank}",
                # the reference's split rule (acc //= gcd(acc, N); batch //= N / gcd) turns this into
                # micro-batch `micro_batch` and `acc` accumulation steps per rank
                "--batch_size", str(a.micro_batch), "--acc_steps", str(acc * (world // a.tp_size)),
                "--scheduler", "cos_inf", "--iterations", str(steps_total),
                "--warmup_steps", "1", "--final_div_factor", "0.1", "--dataset", "fineweb",
                "--datasets_dir", str(data_root), "--log_interval", "1000000", "--eval_interval", "1000000",
                "--latest_ckpt_interval", "0", "--results_base_folder", "/tmp/adana_ref_exps",
                "--run_prefix", f"bench{os.getpid()}"]
        for k, v in OPTS[a.opt].items():
            if isinstance(v, bool):
                if k == "nesterov":
                    argv += ["--nesterov", str(v)]
                elif v:
                    argv.append(f"--{k}")
            else:
                argv += [f"--{k}", str(v)]
        if a.tp_size > 1:
            argv += ["--tp_size", str(a.tp_size)]
        if not a.ref_no_compile:
            argv.append("--compile")
        sys.argv = ["main.py"] + argv
        args, parser = ref_main.get_args()

        # time K optimizer steps from outside: wrap the optimizer's step() of the object the
        # reference builds (the same hook point its own DynamicsLogger uses)
        marks = {"n": 0, "e0": None, "e1": None}
        orig_build = ref_main.build_optimizer

        def build_and_hook(*bargs, **bkw):
            opt = orig_build(*bargs, **bkw)
            orig_step = opt.step

            def timed_step(self_, *sa, **skw):
                r = orig_step(*sa, **skw)
                marks["n"] += 1
                if marks["n"] == a.warmup:
                    torch.cuda.synchronize()
                    if dist.is_initialized():
                        dist.barrier()
                    marks["e0"] = torch.cuda.Event(enable_timing=True)
                    marks["e0"].record()
                    marks["t0"] = time.perf_counter()
                elif marks["n"] == a.warmup + a.steps:
                    marks["e1"] = torch.cuda.Event(enable_timing=True)
                    marks["e1"].record()
                    torch.cuda.synchronize()
                    marks["t1"] = time.perf_counter()
                return r

            import types

            # a bound method, as torch's LR schedulers expect of `optimizer.step`
            opt.step = types.MethodType(timed_step, opt)
            return opt

        ref_main.build_optimizer = build_and_hook
        # keep the process group alive after the reference's main() so the timings can be reduced
        import distributed as ref_dist_pkg
        from distributed import fsdp as ref_fsdp

        ref_fsdp.FSDPDistributedBackend.finalize = lambda self: None
        # the evaluation at iteration 0 / last iteration is not part of the timed region; keep it short
        args.eval_batches = 1
        clocks = None
        from adana_b200.utils.timing import ClockSampler

        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        ref_main.main(args, parser)
        clocks = sampler.stop() if rank == 0 else None
        ms = torch.tensor([marks["e0"].elapsed_time(marks["e1"])], dtype=torch.float64, device=f"cuda:{local_rank}")
        wall = torch.tensor([marks["t1"] - marks["t0"]], dtype=torch.float64, device=f"cuda:{local_rank}")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            dist.all_reduce(wall, op=dist.ReduceOp.MAX)
        ms_per_step = float(ms.item()) / a.steps
        tokens_per_step = a.per_gpu_seqs * (world // a.tp_size) * seq_len
        mem = torch.cuda.max_memory_allocated() / 2 ** 30
        if rank == 0:
            emit({"metric": metric_name(a), "value": tokens_per_step / (ms_per_step / 1e3),
                  "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
                  "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                  "dtype": "bf16 autocast, fp32 parameters", "data": "synthetic Zipf(1.0) tokens, random-init weights",
                  "impl": "reference", "config": shared_config(a, world),
                  "impl_detail": {"compile": not a.ref_no_compile, "attention": "torch SDPA", "fsdp": "torch FSDP2 + NCCL"},
                  "clocks": clocks,
                  "e2e": {"value": tokens_per_step * a.steps / float(wall.item()), "unit": "tokens/s",
                          "h2d_bytes_per_step": 2 * 8 * a.micro_batch * seq_len * acc, "d2h_bytes_per_step": 4,
                          "note": "the reference's own loop: pinned host batches, .item() on the grad norm every step"},
                  "gpu_launches": None, "peak_mem_gib": round(mem, 2)})
        done.set()
        if dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()
    except Exception as e:  # any failure of the reference arm is reported, never raised
        done.set()
        if world > 1:
            note.write_text(f"rank {rank}: {type(e).__name__}: {str(e)[:200]}")
        if rank == 0:
            emit({"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:300]}"})
        else:
            print(f"[reference arm, rank {rank}] {type(e).__name__}: {str(e)[:300]}", file=sys.stderr, flush=True)


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
