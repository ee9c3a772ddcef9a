import argparse

import pytest

from adana_b200.config import compute_dimensions, compute_lr, flags
from adana_b200.config.scaling import apply_scaling_rule
from adana_b200.main import get_args, get_exp_name


def test_scaling_dimensions():
    d = compute_dimensions("enoki", 36)
    assert (d["n_layer"], d["n_embd"], d["mlp_hidden_dim"], d["qkv_dim"]) == (27, 2304, 9216, 64)
    assert d["non_emb_params"] == 12 * 2304 ** 2 * 27
    assert d["total_params"] == d["non_emb_params"] + 2 * 2304 * 50304
    q = compute_dimensions("qwen3", 16)
    assert (q["n_layer"], q["n_embd"], q["mlp_hidden_dim"], q["qkv_dim"]) == (32, 2048, 6144, 128)
    e3 = compute_dimensions("enoki", 3)
    assert (e3["n_layer"], e3["n_embd"]) == (2, 192)
    with pytest.raises(ValueError):
        compute_dimensions("nope", 4)


def test_lr_laws():
    P = 12 * 768 ** 2 * 9
    assert compute_lr("enoki", "adamw", P) == pytest.approx(12.8 * (1.67e4 + P) ** -0.515)
    assert compute_lr("enoki", "dana-star-mk4", P, kappa=0.85) == pytest.approx(223.0 * (2.40e6 + P) ** -0.724)
    # closest-kappa fallback and the batch-512 table with fallback to the batch-32 one
    assert compute_lr("enoki", "adana", P, kappa=0.82) == pytest.approx(17.6 * (3.66e4 + P) ** -0.624)
    assert compute_lr("enoki", "adana", P, kappa=0.85, batch_size=512) == pytest.approx(85.3 * (3.04e4 + P) ** -0.654)
    assert compute_lr("enoki", "d-muon", P, batch_size=512) == pytest.approx(2.19 * (5.64e4 + P) ** -0.417)
    assert compute_lr("enoki", "lion", P) is None
    assert compute_lr("qwen3", "adamw", P) == pytest.approx(2.16e4 * (7.20e4 + P) ** -0.873)


def test_apply_scaling_rule_sets_shape_lr_iterations():
    a = flags.defaults()
    a.scaling_rule, a.heads, a.opt, a.kappa = "enoki", 12, "dana-mk4", 0.85
    a.batch_size, a.acc_steps, a.sequence_length = 32, 1, 2048
    apply_scaling_rule(a, verbose=False)
    assert (a.model, a.n_layer, a.n_embd, a.n_head, a.weight_tying) == ("enoki", 9, 768, 12, False)
    total = 12 * 768 ** 2 * 9 + 2 * 768 * 50304
    assert a.iterations == int(20 * total / (32 * 2048))
    assert a.lr == pytest.approx(23.0 * (1.46e4 + 12 * 768 ** 2 * 9) ** -0.627)


def test_flag_surface_and_aliases():
    args, parser = get_args(["--model", "enoki", "--opt", "dana-star-mk4", "--distributed_backend", "ddp",
                             "--init-scheme", "ScaledGPT", "--residual-stream-scalar", "0.5", "--no-qknorm",
                             "--collect-tau-stats", "--weight_tying", "False", "--nesterov", "True",
                             "--iterations", "1000", "--kappa", "0.85"])
    assert args.distributed_backend == "nccl" and args.init_scheme == "ScaledGPT" and args.no_qknorm
    assert args.residual_stream_scalar == 0.5 and args.collect_tau_stats and args.weight_tying is False
    assert args.nesterov is True and args.full_eval_at == []
    assert args.adema_beta3 == pytest.approx(1 - 8.0 / 1000) and args.adema_alpha == pytest.approx(1000 ** 0.15)
    assert len(flags.OPTIMIZERS) == 24
    with pytest.raises(SystemExit):
        get_args(["--opt", "not-an-optimizer"])
    with pytest.raises(ValueError):
        get_args(["--tp_size", "2", "--distributed_backend", "nccl"])


def test_exp_name():
    args, parser = get_args(["--model", "enoki", "--opt", "adana", "--dataset", "fineweb", "--batch_size", "32",
                             "--lr", "0.002", "--seed", "3", "--wandb"])
    name = get_exp_name(args, parser)
    assert name.startswith("32x1_model-enoki_dataset-fineweb_opt-adana__")
    assert "lr-0.002" in name and "seed" not in name and "wandb" not in name
    args.run_prefix = "x" * 250
    assert "__hash_" in get_exp_name(args, parser)


def test_scaling_rules_equal_the_reference_functions(ref_src):
    """Model dimensions, learning-rate laws (every optimizer table, kappa keys and the closest-kappa fallback, the
    batch-512 table) and `apply_scaling_rule` against the reference's own functions over a grid: same values, and
    the same error where the reference raises."""
    import contextlib
    import copy
    import importlib.util
    import io
    import itertools

    from adana_b200.config import flags
    from adana_b200.config import scaling as mine

    spec = importlib.util.spec_from_file_location("ref_scaling", ref_src / "config" / "scaling.py")
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)

    def outcome(fn, *a, **k):
        try:
            return fn(*a, **k)
        except Exception as e:      # the error class is part of the behaviour
            return ("error", type(e).__name__)

    for rule, heads in itertools.product(("enoki", "qwen3"), (4, 8, 12, 16, 24, 28, 32, 36, 44, 48)):
        a, b = mine.compute_dimensions(rule, heads), ref.compute_dimensions(rule, heads)
        assert {k: a.get(k) for k in b} == b, (rule, heads)
    opts = ("adamw", "adamw-decaying-wd", "adana", "dana-mk4", "dana-star", "dana-star-mk4", "dana-star-mk4-tau", "ademamix",
            "ademamix-decaying-wd", "d-muon", "lion")
    for rule, opt, kappa, bs, P in itertools.product(("enoki", "qwen3"), opts, (None, 0.75, 0.8, 0.85, 0.9, 0.83),
                                                     (None, 32, 512), (1e7, 2.5e9)):
        x = outcome(mine.compute_lr, rule, opt, P, kappa=kappa, batch_size=bs)
        y = outcome(ref.compute_lr, rule, opt, P, kappa=kappa, batch_size=bs)
        assert x == y or (isinstance(x, float) and isinstance(y, float) and abs(x - y) <= 1e-12 * abs(y)), (rule, opt, kappa, bs, P, x, y)
    for rule, opt, heads, B, acc in itertools.product(("enoki", "qwen3"), ("adamw", "dana-star-mk4", "d-muon"), (8, 36), (32, 64), (1, 8)):
        a = flags.defaults()
        a.scaling_rule, a.opt, a.heads, a.kappa, a.batch_size, a.acc_steps = rule, opt, heads, 0.85, B, acc
        x, y = copy.deepcopy(a), copy.deepcopy(a)
        with contextlib.redirect_stdout(io.StringIO()):
            mine.apply_scaling_rule(x)
            ref.apply_scaling_rule(y)
        assert vars(x) == vars(y), (rule, opt, heads, B, acc)


def test_flag_surface_and_defaults_equal_the_reference_parser(ref_src):
    """Every flag of the reference's parser exists here with the same default; the two that differ are paths into
    the reference's own source tree."""
    import argparse
    import importlib.util
    import sys
    import types

    from adana_b200.config import flags

    had = "distributed" in sys.modules
    if not had:     # the reference's config imports its distributed package only for the backend names
        sys.modules["distributed"] = types.SimpleNamespace(registered_backends=lambda: ["nccl", "gloo", "fsdp"])
    try:
        spec = importlib.util.spec_from_file_location("ref_config_base", ref_src / "config" / "base.py")
        ref = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ref)
        want = vars(ref.parse_args(argparse.ArgumentParser(allow_abbrev=False), args=[], namespace=None))
    finally:
        if not had:
            del sys.modules["distributed"]
    got = vars(flags.defaults())
    assert not set(want) - set(got)
    different = {k for k in want if got[k] != want[k]}
    assert different == {"dynamics_logger_cfg", "datasets_dir"}, different


def test_experiment_directory_names_equal_the_reference(ref_src, monkeypatch):
    """`get_exp_name` against the reference's function, the md5 tag of over-long names included: a run started with
    one code base is found by `--auto_resume` of the other."""
    import argparse
    import importlib
    import sys
    import types

    import tiktoken
    import torch

    from adana_b200 import main as ours
    from adana_b200.config import parse_args_with_format

    torch.compiler.set_stance("force_eager")
    monkeypatch.setattr(tiktoken, "get_encoding", lambda name: types.SimpleNamespace(name=name))
    top = ("config", "models", "optim", "data", "distributed", "logger", "main")

    def forget():
        for k in [k for k in sys.modules if k.split(".")[0] in top]:
            del sys.modules[k]

    cases = [[], ["--model", "enoki", "--opt", "dana-star-mk4", "--lr", "0.002", "--kappa", "0.8"],
             ["--batch_size", "64", "--acc_steps", "8", "--n_layer", "36", "--distributed_backend", "fsdp"],
             ["--opt", "adamw", "--weight_decay", "0.01", "--run_prefix", "abc", "--seed", "3", "--wd_decaying", "--wd_ts", "17"],
             ["--model", "qwen3", "--moe", "--moe_num_experts", "16", "--z_loss_coeff", "0.001", "--scheduler", "wsd",
              "--wsd_fract_decay", "0.2", "--dataset", "fineweb_100", "--sequence_length", "2048", "--n_embd", "2304",
              "--n_head", "36", "--mlp_hidden_dim", "9216", "--qkv_dim", "64", "--iterations", "12345", "--warmup_steps",
              "246", "--grad_clip", "0.5", "--delta", "8", "--clipsnr", "2.0", "--eval_interval", "115"]]
    forget()
    if "wandb" not in sys.modules:
        try:
            import wandb  # noqa: F401
        except Exception:
            monkeypatch.setitem(sys.modules, "wandb", types.ModuleType("wandb"))
    sys.path.insert(0, str(ref_src))
    try:
        ref_main = importlib.import_module("main")
        ref_config = importlib.import_module("config")
        want = []
        for argv in cases:
            p = argparse.ArgumentParser(allow_abbrev=False)
            p.add_argument("--config_format", default="base")
            a = ref_config.parse_args_with_format(format="base", base_parser=p, namespace=None, args=argv)
            want.append(ref_main.get_exp_name(a, p, types.SimpleNamespace(rank=0)))
    finally:
        sys.path.remove(str(ref_src))
        forget()
    for argv, w in zip(cases, want):
        p = argparse.ArgumentParser(allow_abbrev=False)
        p.add_argument("--config_format", default="base")
        a = parse_args_with_format(format="base", base_parser=p, namespace=None, args=argv)
        assert ours.get_exp_name(a, p, None) == w
    assert "__hash_" in want[-1]
