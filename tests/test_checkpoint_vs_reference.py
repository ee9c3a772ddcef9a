"""Checkpoint interchange with the reference: a `main.pt` written by the reference's `save_checkpoint` (its model,
its ADana-family optimizer, its scheduler) is resumed here, through the autograd path and through the kernel
engine, and a checkpoint written here is resumed by the reference's `load_checkpoint`; after the switch both sides
follow the same loss curve.  Needs the unmodified reference under baseline/_ref."""
import argparse
import sys
import types

import pytest
import torch

ARGV = ["--model", "enoki", "--n_layer", "2", "--n_head", "2", "--n_embd", "128", "--qkv_dim", "64", "--mlp_hidden_dim",
        "256", "--sequence_length", "32", "--batch_size", "4", "--vocab_size", "512", "--dtype", "float32", "--device",
        "cpu", "--dropout", "0.0", "--z_loss_coeff", "1e-3", "--weight_tying", "False"]
OPT_KW = dict(lr=2e-3, delta=8.0, kappa=0.85, weight_decay=0.2, clipsnr=2.0, wd_decaying=True, wd_ts=5.0, gamma_3_factor=1.0)
STEPS, SWITCH, TOTAL = 12, 4, 8
_TOP = ("config", "models", "optim", "data", "distributed", "logger")


def _batches():
    g = torch.Generator().manual_seed(11)
    return [(torch.randint(0, 512, (4, 32), generator=g), torch.randint(0, 512, (4, 32), generator=g)) for _ in range(TOTAL)]


class _Reference:
    """The reference's packages imported under their own top-level names for the duration of a `with` block."""

    def __init__(self, ref_src, monkeypatch):
        self.src, self.mp = str(ref_src), monkeypatch

    def _forget(self):
        for k in [k for k in sys.modules if k.split(".")[0] in _TOP]:
            del sys.modules[k]

    def __enter__(self):
        import tiktoken

        torch.compiler.set_stance("force_eager")
        self.mp.setattr(tiktoken, "get_encoding", lambda name: types.SimpleNamespace(name=name))
        if "wandb" not in sys.modules:
            try:
                import wandb  # noqa: F401
            except Exception:
                self.mp.setitem(sys.modules, "wandb", types.ModuleType("wandb"))
        self._forget()
        sys.path.insert(0, self.src)
        import config
        from models.utils import get_model
        from optim.dana_star_mk4 import DANA_STAR_MK4
        from optim.schedule import cos_inf_schedule
        from optim.utils import load_checkpoint, save_checkpoint

        self.config, self.get_model, self.opt_cls = config, get_model, DANA_STAR_MK4
        self.sched_fn, self.load, self.save = cos_inf_schedule, load_checkpoint, save_checkpoint
        return self

    def __exit__(self, *exc):
        sys.path.remove(self.src)
        self._forget()

    def build(self):
        p = argparse.ArgumentParser(allow_abbrev=False)
        p.add_argument("--config_format", default="base")
        torch.manual_seed(0)
        model = self.get_model(self.config.parse_args_with_format(format="base", base_parser=p, namespace=None, args=ARGV))
        named = dict(model.named_parameters())
        specs = model.get_parameter_group_specs()
        for g in specs:
            g["params"] = [named[n] for n in g["params"]]
        opt = self.opt_cls(specs, **OPT_KW)
        sched = torch.optim.lr_scheduler.LambdaLR(opt, self.sched_fn(STEPS, 3, 1e2, 1e4, 0))
        return model, opt, sched


def _ours(engine):
    from adana_b200.config import parse_args_with_format
    from adana_b200.models.utils import get_model
    from adana_b200.optim.logtime import DanaStarMK4
    from adana_b200.optim.schedule import CosInf

    p = argparse.ArgumentParser(allow_abbrev=False)
    p.add_argument("--config_format", default="base")
    args = parse_args_with_format(format="base", base_parser=p, namespace=None, args=ARGV)
    torch.manual_seed(1)
    model = get_model(args)
    specs = model.get_parameter_group_specs()
    eng = None
    if engine:
        from adana_b200.runtime.engine import EngineOptimizer, attach

        for k, v in dict(opt="dana-star-mk4", acc_steps=1, **OPT_KW).items():
            setattr(args, k, v)
        args.gamma_3_factor = OPT_KW["gamma_3_factor"]
        eng = attach(model, args, device="cpu")
        for g in specs:
            g["param_names"] = g["params"]
        opt = EngineOptimizer(eng, "dana-star-mk4", args, specs)
    else:
        named = dict(model.named_parameters())
        for g in specs:
            g["params"] = [named[n] for n in g["params"]]
        opt = DanaStarMK4(specs, **OPT_KW)
    sched = torch.optim.lr_scheduler.LambdaLR(opt, CosInf(STEPS, 3, 1e2, 1e4, 0))
    return model, opt, sched, eng


def _train(model, opt, sched, batches, eng=None):
    model.train()
    losses = []
    for x, y in batches:
        out = model(x, targets=y)
        out["loss"].backward()
        if eng is not None:
            eng.grad_norm_and_clip(0.5)
        else:
            torch.nn.utils.clip_grad_norm_(model.parameters(), 0.5)
        opt.step()
        sched.step()
        opt.zero_grad(set_to_none=True)
        losses.append(out["loss"].item())
    return losses


@pytest.mark.parametrize("engine", [False, True], ids=["autograd", "engine"])
def test_reference_checkpoint_resumes_here(ref_src, monkeypatch, tmp_path, engine):
    from adana_b200.train.checkpoint import load_checkpoint

    batches = _batches()
    with _Reference(ref_src, monkeypatch) as ref:
        model, opt, sched = ref.build()
        _train(model, opt, sched, batches[:SWITCH])
        ref.save(model, opt, sched, SWITCH, tmp_path / "ckpt")
        want = _train(model, opt, sched, batches[SWITCH:])
    model, opt, sched, eng = _ours(engine)
    assert load_checkpoint(model, opt, sched, tmp_path / "ckpt" / "main.pt") == SWITCH
    got = _train(model, opt, sched, batches[SWITCH:], eng)
    for a, b in zip(got, want):
        assert a == pytest.approx(b, rel=2e-5), (got, want)


@pytest.mark.parametrize("engine", [False, True], ids=["autograd", "engine"])
def test_checkpoint_written_here_resumes_in_the_reference(ref_src, monkeypatch, tmp_path, engine):
    from adana_b200.train.checkpoint import save_checkpoint

    batches = _batches()
    with _Reference(ref_src, monkeypatch) as ref:       # same initial weights on both sides
        init = {k: v.clone() for k, v in ref.build()[0].state_dict().items()}
    model, opt, sched, eng = _ours(engine)
    if eng is not None:
        eng.load_full_param_dict(init)
    else:
        model.load_state_dict(init)
    _train(model, opt, sched, batches[:SWITCH], eng)
    save_checkpoint(model, opt, sched, SWITCH, tmp_path / "ckpt")
    want = _train(model, opt, sched, batches[SWITCH:], eng)
    with _Reference(ref_src, monkeypatch) as ref:
        model, opt, sched = ref.build()
        assert ref.load(model, opt, sched, tmp_path / "ckpt" / "main.pt", "cpu") == SWITCH
        got = _train(model, opt, sched, batches[SWITCH:])
    for a, b in zip(got, want):
        assert a == pytest.approx(b, rel=2e-5), (got, want)


def test_worker_state_files_are_interchangeable(ref_src, monkeypatch, tmp_path):
    """`worker_0.pt` (RNG states + data reader position) written by either side is restored by the other: the next
    batches and the next random numbers are the ones the writer would have produced."""
    import importlib
    import random

    import numpy as np

    from adana_b200.data.readers import DataReader
    from adana_b200.train import checkpoint as ours

    toks = np.random.default_rng(0).integers(0, 50000, size=60000).astype(np.uint16)
    kw = dict(local_batch_size=4, sequence_length=32, seed=5, keep_in_ram=True, with_replacement=False, auto_shard=False)
    with _Reference(ref_src, monkeypatch):
        ref_utils = importlib.import_module("optim.utils")
        ref_reader_cls = importlib.import_module("data.utils").DataReader
        # reference writes, this side restores
        r = ref_reader_cls(toks, **kw)
        r.set_step(0)
        for _ in range(7):
            r.sample_batch()
        torch.manual_seed(3)
        np.random.seed(4)
        random.seed(5)
        ref_utils.save_worker_state(tmp_path / "a", r)
        want = (r.sample_batch()[0], torch.rand(3), np.random.rand(), random.random())
        m = DataReader(toks, **kw)
        torch.manual_seed(99)
        ours.load_worker_state(tmp_path / "a", m, verbose=False)
        got = (m.sample_batch()[0], torch.rand(3), np.random.rand(), random.random())
        assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1]) and got[2:] == want[2:]
        # this side writes, the reference restores
        for _ in range(5):
            m.sample_batch()
        ours.save_worker_state(tmp_path / "b", m, verbose=False)
        want = (m.sample_batch()[0], torch.rand(3), np.random.rand(), random.random())
        r2 = ref_reader_cls(toks, **kw)
        torch.manual_seed(98)
        ref_utils.load_worker_state(tmp_path / "b", r2)
        got = (r2.sample_batch()[0], torch.rand(3), np.random.rand(), random.random())
        assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1]) and got[2:] == want[2:]
