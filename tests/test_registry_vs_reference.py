"""`--opt NAME` wiring against the reference: for every optimizer name the class built by `build_optimizer` and the
hyper-parameters in its parameter groups (what `state_dict()["param_groups"]` carries in a checkpoint) must equal
those the reference's `build_optimizer` produces from the same command line (its `get_args` derivations included)."""
import sys
import types

import pytest
import torch

NAMES = ["adamw", "sgd", "ademamix", "ademamix-decaying-wd", "adamw-decaying-wd", "lion", "sf-adamw", "sf-sgd", "signsgd",
         "signum", "prodigy", "sophiag", "adopt", "mars", "adafactor", "lamb", "adana", "dana-mk4", "dana-star",
         "dana-star-mk4", "soap", "muon", "d-muon", "manau"]
BASE = ["--iterations", "1000", "--warmup_steps", "20", "--lr", "0.002", "--weight_decay", "0.05", "--kappa", "0.8",
        "--clipsnr", "1.5", "--wd_ts", "7", "--wd_decaying", "--device", "cpu"]
# torch's own bookkeeping switches, which depend on the torch version rather than on the wiring
TORCH_KEYS = {"foreach", "fused", "capturable", "maximize", "differentiable", "decoupled_weight_decay"}
CLASS_ALIASES = {"DANA_STAR_MK4": "DanaStarMK4", "AdEMAMix_DecayingWD": "AdEMAMixDecayingWD"}
_TOP = ("config", "models", "optim", "data", "distributed", "logger", "main")


def _problem():
    torch.manual_seed(0)
    m = torch.nn.Sequential(torch.nn.Linear(8, 16, bias=False), torch.nn.Linear(16, 4, bias=False))
    named = dict(m.named_parameters())
    return m, [{"params": [named["0.weight"]], "param_names": ["transformer.h.0.mlp.c_fc.weight"]},
               {"params": [named["1.weight"]], "param_names": ["transformer.h.0.ln_1.weight"], "weight_decay": 0.0}]


def _groups(opt):
    return [{k: v for k, v in g.items() if k not in ("params", "param_names") and k not in TORCH_KEYS} for g in opt.param_groups]


@pytest.fixture(scope="module")
def reference_builds(ref_src):
    import importlib

    import tiktoken

    torch.compiler.set_stance("force_eager")
    saved_enc, saved_argv = tiktoken.get_encoding, sys.argv
    tiktoken.get_encoding = lambda name: types.SimpleNamespace(name=name)
    added_wandb = False
    if "wandb" not in sys.modules:
        try:
            import wandb  # noqa: F401
        except Exception:
            sys.modules["wandb"] = types.ModuleType("wandb")
            added_wandb = True
    for k in [k for k in sys.modules if k.split(".")[0] in _TOP]:
        del sys.modules[k]
    sys.path.insert(0, str(ref_src))
    out = {}
    try:
        ref_main = importlib.import_module("main")
        for name in NAMES:
            sys.argv = ["main.py", *BASE, "--opt", name]
            args, _ = ref_main.get_args()
            model, specs = _problem()
            opt = ref_main.build_optimizer(args, model, specs)
            out[name] = (type(opt).__name__, _groups(opt))
    finally:
        sys.argv = saved_argv
        tiktoken.get_encoding = saved_enc
        sys.path.remove(str(ref_src))
        for k in [k for k in sys.modules if k.split(".")[0] in _TOP]:
            del sys.modules[k]
        if added_wandb:
            del sys.modules["wandb"]
    return out


@pytest.mark.parametrize("name", NAMES)
def test_optimizer_built_from_flags_equals_the_reference(reference_builds, name):
    from adana_b200.main import get_args
    from adana_b200.optim.registry import build_optimizer

    args, _ = get_args([*BASE, "--opt", name])
    model, specs = _problem()
    opt = build_optimizer(args, model, specs)
    want_cls, want_groups = reference_builds[name]
    assert type(opt).__name__ == CLASS_ALIASES.get(want_cls, want_cls)
    got_groups = _groups(opt)
    assert len(got_groups) == len(want_groups)
    for got, want in zip(got_groups, want_groups):
        assert set(got) == set(want), (name, set(got) ^ set(want))
        for k in want:
            assert got[k] == want[k], (name, k, got[k], want[k])
