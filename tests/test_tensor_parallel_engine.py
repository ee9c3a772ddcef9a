"""Tensor parallelism on the kernel engine, on CPU ranks over Gloo: dp x tp runs equal the single-process run (same
batches per data-parallel replica), for both architectures, with the sums over tp taken by `torch.distributed`."""
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "tests"))
from test_distributed_cpu import _spawn, _t  # noqa: E402


def _args(model):
    from conftest import tiny_args

    kw = dict(n_kv_head=2) if model == "qwen3" else dict(multiple_of=32) if model == "llama" else {}
    return tiny_args(model, n_head=4, n_embd=128, qkv_dim=32, mlp_hidden_dim=256, opt="dana-star-mk4", kappa=0.85,
                     clipsnr=2.0, lr=2e-3, weight_decay=0.1, wd_decaying=True, wd_ts=3.0, acc_steps=1, grad_clip=0.5, **kw)


def _run(model, comm, tp_group, dp_rank, dp_size, steps=3):
    from adana_b200.models.utils import get_model
    from adana_b200.runtime.engine import EngineOptimizer, attach

    a = _args(model)
    torch.manual_seed(0)
    m = get_model(a)
    eng = attach(m, a, comm=comm, sharded=True, device="cpu", tp_group=tp_group)
    specs = m.get_parameter_group_specs()
    for g in specs:
        g["param_names"] = g["params"]
    opt = EngineOptimizer(eng, a.opt, a, specs)
    m.train()
    losses, norms = [], []
    for step in range(steps):
        tot = 0.0
        # the single process sees every replica's batch in turn (gradient accumulation = data parallelism)
        replicas = range(2) if dp_size == 0 else [dp_rank]
        for i, r in enumerate(replicas):
            g = torch.Generator().manual_seed(100 * step + r)
            idx = torch.randint(0, a.vocab_size, (2, a.sequence_length), generator=g)
            eng.sync_on_backward = i == len(replicas) - 1
            eng.loss_scale = 1.0 / len(replicas)
            out = m(idx, targets=idx.roll(-1, 1))
            (out["loss"] / len(replicas)).backward()
            tot += out["loss"].item() / len(replicas)
        norms.append(float(eng.grad_norm_and_clip(0.5)))
        opt.step()
        opt.zero_grad()
        losses.append(tot)
    full = eng.full_param_dict("master")
    return {"losses": losses, "norms": norms, "params": {k: v.clone() for k, v in full.items()},
            "local_qkv_rows": eng.units[0].layout.slots[0].shape[0]}


def _tp_worker(rank, world, model, tp):
    from adana_b200.parallel.comm import Comm

    dist.init_process_group("gloo")
    dp = world // tp
    tp_group = dp_group = None
    for i in range(dp):
        ranks = list(range(i * tp, (i + 1) * tp))
        g = dist.new_group(ranks)
        if rank in ranks:
            tp_group = g
    for j in range(tp):
        ranks = list(range(j, world, tp))
        g = dist.new_group(ranks)
        if rank in ranks:
            dp_group = g
    return _run(model, Comm(dp_group), tp_group, rank // tp, dp)


def _single(model, replicas):
    from adana_b200.parallel.comm import Comm

    return _run(model, Comm(), None, 0, 0 if replicas == 2 else 1)


@pytest.mark.parametrize("model,world,tp", [("enoki", 2, 2), ("qwen3", 2, 2), ("enoki", 4, 2), ("llama", 2, 2)])
def test_tensor_parallel_engine_equals_single_process(model, world, tp):
    res = _spawn(_tp_worker, world, model, tp)
    ref = _single(model, world // tp)
    for r in range(world):
        got = res[r]
        assert got["local_qkv_rows"] * tp == ref["local_qkv_rows"] or model == "qwen3"
        assert ("lm_head.weight" in got["params"]) == ("lm_head.weight" in ref["params"])
        for x, y in zip(got["losses"], ref["losses"]):
            assert abs(x - y) < 2e-5 * abs(y) + 1e-6 or world // tp > 1, (got["losses"], ref["losses"])
        for x, y in zip(got["norms"], ref["norms"]):
            assert abs(x - y) < 1e-4 * y, (got["norms"], ref["norms"])
        for k, v in ref["params"].items():
            assert tuple(_t(got["params"][k]).shape) == tuple(v.shape), k
            # (the update divides by a running second moment: where a gradient is next to zero the last bits decide its
            # size, so a handful of elements may differ by a fraction of the learning rate)
            d = (_t(got["params"][k]) - v).abs()
            assert d.mean().item() < 2e-6 and (d > 1e-5).float().mean().item() < 5e-3 and d.max().item() < 2e-3, \
                (k, d.mean().item(), d.max().item())


def test_slicing_rules_round_trip_and_reject_indivisible_heads():
    from adana_b200.models.utils import get_model
    from adana_b200.parallel.tensor_parallel import check_divisible, shard_model_for_tp, tp_unslice

    for model in ("enoki", "qwen3", "llama"):
        a = _args(model)
        torch.manual_seed(0)
        full = {k: v.detach().clone() for k, v in get_model(a).named_parameters()}
        parts = []
        for r in range(2):
            torch.manual_seed(0)
            m = get_model(a)
            cut = shard_model_for_tp(m, r, 2)
            parts.append(dict(m.named_parameters()))
        assert len(cut) == a.n_layer * {"enoki": 4, "qwen3": 7, "llama": 5}[model]
        for name, rule in cut.items():
            assert torch.equal(tp_unslice([parts[0][name].data, parts[1][name].data], rule), full[name])
        with pytest.raises(ValueError, match="not divisible"):
            check_divisible(get_model(a), 3)
