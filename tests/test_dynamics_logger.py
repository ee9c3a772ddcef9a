"""Dynamics logger: statistic values against closed forms, interval schedule, disk round trip, engine source."""
import math

import torch

from conftest import tiny_args
from adana_b200.logging.dynamics import STATS, DynamicsLogger, load_logger_config


def _toy():
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(6, 4), torch.nn.Linear(4, 2))
    opt = torch.optim.AdamW(model.parameters(), lr=0.05, weight_decay=0.0)
    return model, opt


def test_statistics_match_closed_forms(tmp_path):
    model, opt = _toy()
    cfg = load_logger_config(None)
    cfg.update(interval=1, stats=sorted(STATS), disk_save_interval=None, wandb_interval=None)
    lg = DynamicsLogger(model, opt, cfg, tmp_path)
    x = torch.randn(8, 6)
    model(x).square().mean().backward()
    w0 = model[0].weight.detach().clone()
    g0 = model[0].weight.grad.detach().clone()
    b0 = model[0].bias.detach().clone()
    opt.step()
    w1 = model[0].weight.detach()
    s = lg.stats
    assert torch.allclose(s["layer_norm"]["0.weight"][0], w0.norm())
    assert torch.allclose(s["neuron_norm"]["0.weight"][0], w0.norm(dim=1))
    assert torch.allclose(s["layer_grad_norm"]["0.weight"][0], g0.norm())
    assert torch.allclose(s["neuron_update_norm"]["0.weight"][0], (w1 - w0).norm(dim=1))
    rel = ((w1 - w0).norm() + 1e-8) / (w0.norm() + 1e-8)
    assert torch.allclose(s["layer_relative_update"]["0.weight"][0], rel)
    cos = torch.nn.functional.cosine_similarity(w0.double().flatten(), w1.double().flatten(), dim=0)
    assert math.isclose(float(s["layer_angular_update"]["0.weight"][0]), math.acos(min(1.0, float(cos))), rel_tol=1e-4)
    assert torch.allclose(s["scalar_rms"]["0.bias"][0], b0.square().mean().sqrt())
    assert "0.bias" not in s["layer_norm"] and "0.weight" not in s["scalar_rms"]
    # first Adam step: v = (1-b2) g², so g / sqrt(v) has a known norm
    v = (1 - 0.999) * g0.square()
    assert torch.allclose(s["layer_scaled_grad_norm"]["0.weight"][0], (g0 / (v.sqrt() + 1e-8)).norm(), rtol=1e-4)
    # no first moment existed before the first step: alignment is reported as zero
    assert float(s["layer_grad_velocity_alignment"]["0.weight"][0]) == 0.0
    model.zero_grad()
    model(x).square().mean().backward()
    g1 = model[0].weight.grad.detach().clone()
    m1 = opt.state[model[0].weight]["exp_avg"].clone()
    opt.step()
    want = torch.nn.functional.cosine_similarity(g1.flatten(), m1.flatten(), dim=0)
    assert torch.allclose(s["layer_grad_velocity_alignment"]["0.weight"][1], want, atol=1e-6)


def test_interval_schedule_and_disk_round_trip(tmp_path):
    model, opt = _toy()
    cfg = load_logger_config(None)
    cfg.update(interval=[(0, 1), (4, 2)], stats=["layer_norm", "neuron_norm", "scalar_rms"], disk_save_interval=2,
               disk_downsample=2, disk_max_channels=3, wandb_interval=None)
    lg = DynamicsLogger(model, opt, cfg, tmp_path)
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda i: 1.0)     # schedulers wrap step() after the logger
    logged = []
    for it in range(8):
        model.zero_grad()
        model(torch.randn(8, 6)).square().mean().backward()
        before = sum(len(v) for v in lg.stats["layer_norm"].values())
        opt.step()
        sched.step()
        after = sum(len(v) for v in lg.stats["layer_norm"].values())
        logged.append(after != before or (tmp_path / "dynamics.pkl").exists() and after < before)
    assert lg.iteration == 8
    stats = DynamicsLogger.load_stats(tmp_path / "dynamics.pkl")
    assert set(stats) == {"layer_norm", "neuron_norm", "scalar_rms"}
    assert stats["neuron_norm"]["0.weight"].shape[1] == 3            # channel cap
    assert stats["layer_norm"]["0.weight"].shape[0] >= 2             # one down-sampled row per flush
    assert torch.isfinite(stats["scalar_rms"]["1.bias"]).all()


def test_engine_source_reports_updates_of_flat_buffers(tmp_path):
    from adana_b200.models.utils import get_model
    from adana_b200.runtime.engine import EngineOptimizer, attach

    a = tiny_args("enoki", opt="adamw", lr=1e-2, weight_decay=0.0, acc_steps=1, grad_clip=0.0)
    torch.manual_seed(0)
    m = get_model(a)
    eng = attach(m, a, device="cpu")
    specs = m.get_parameter_group_specs()
    for g in specs:
        g["param_names"] = g["params"]
    opt = EngineOptimizer(eng, "adamw", a, specs)
    cfg = load_logger_config(None)
    cfg.update(interval=1, stats=["layer_update_norm", "layer_grad_norm", "scalar_update_rms", "layer_mean_second_grad_moment"],
               wandb_interval=None)
    lg = DynamicsLogger(m, opt, cfg, tmp_path)
    idx = torch.randint(0, a.vocab_size, (2, a.sequence_length))
    m.train()
    m(idx, targets=idx.roll(-1, 1))["loss"].backward()
    opt.step()
    name = "transformer.h.0.attn.c_attn.weight"
    n = m.transformer.h[0].attn.c_attn.weight.numel()
    # first AdamW step moves every element by ~lr
    assert abs(float(lg.stats["layer_update_norm"][name][0]) / (1e-2 * math.sqrt(n)) - 1) < 0.05
    assert float(lg.stats["layer_grad_norm"][name][0]) > 0
    assert float(lg.stats["layer_mean_second_grad_moment"][name][0]) > 0
    assert any(float(v[0]) > 0 for v in lg.stats["scalar_update_rms"].values())


def test_disk_output_equals_the_reference_logger(ref_src, tmp_path):
    """Same model, same optimizer, same steps, the reference's YAML configuration: the `dynamics.pkl` written by
    the reference's DynamicsLogger and by this one hold the same statistics for the same parameters.  One is
    excluded: the reference's `scalar_rms` reads a stale loop variable (src/logger/logger.py:117,271: the model's
    last parameter, whatever the scalar being logged), here it is the RMS of the parameter itself."""
    import copy
    import importlib.util

    import yaml

    from adana_b200.logging.dynamics import DynamicsLogger

    spec = importlib.util.spec_from_file_location("ref_logger", ref_src / "logger" / "logger.py")
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    cfg = yaml.safe_load((ref_src / "logger" / "rotational_logger.yaml").read_text())
    cfg.update(interval=1, disk_save_interval=4, disk_downsample=2, wandb_interval=None)
    out = {}
    for name, cls in (("ref", ref.DynamicsLogger), ("ours", DynamicsLogger)):
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(12, 24, bias=True), torch.nn.LayerNorm(24), torch.nn.Linear(24, 6, bias=False))
        opt = torch.optim.AdamW(model.parameters(), lr=1e-2, weight_decay=0.1)
        folder = tmp_path / name
        folder.mkdir()
        cls(model, opt, copy.deepcopy(cfg), folder, wandb=False)
        g = torch.Generator().manual_seed(1)
        for _ in range(8):
            loss = model(torch.randn(16, 12, generator=g)).pow(2).mean()
            opt.zero_grad()
            loss.backward()
            opt.step()
        out[name] = cls.load_stats(folder / "dynamics.pkl")
    want, got = out["ref"], out["ours"]
    assert set(want) == set(got) == set(cfg["stats"])
    for stat in want:
        assert set(want[stat]) == set(got[stat]), stat
        if stat == "scalar_rms":
            continue
        for pname in want[stat]:
            assert got[stat][pname].shape == want[stat][pname].shape == torch.Size([4, got[stat][pname].shape[1]])
            assert got[stat][pname].dtype == want[stat][pname].dtype, (stat, pname, got[stat][pname].dtype, want[stat][pname].dtype)
            # an angle of 0.05 rad moves by 1e-6 when an operand moves by one fp32 ulp
            rtol = 1e-4 if "angular" in stat else 1e-5
            assert torch.allclose(got[stat][pname], want[stat][pname], atol=1e-6, rtol=rtol), (stat, pname)
