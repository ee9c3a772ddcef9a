import math

import pytest
import torch

from adana_b200.optim.schedule import CosInf, PowerLaw, WSD, build_scheduler, cos_inf_schedule, wsd_schedule


def test_cos_inf():
    s = cos_inf_schedule(1000, 100, 100.0, 0.1, 0)
    assert s(0) == pytest.approx(0.01)
    assert s(50) == pytest.approx(0.5 + 0.5 / 100)
    assert s(100) == pytest.approx(1.0)
    floor = 1 / 100 / 0.1
    assert s(550) == pytest.approx(floor + 0.5 * (1 - floor))
    assert s(1000) == pytest.approx(floor) and s(5000) == pytest.approx(floor)
    s2 = CosInf(1000, 100, 100.0, 1.0, 200)
    assert s2(800) == pytest.approx(0.01) and s2(799) > 0.01


@pytest.mark.parametrize("kind", ["linear", "exp", "cosine", "miror_cosine", "square", "sqrt"])
def test_wsd_shapes(kind):
    s = wsd_schedule(1000, final_lr_factor=0.1, n_warmup=100, init_div_factor=100, fract_decay=0.2, decay_type=kind)
    assert s(0) == pytest.approx(0.01) and s(100) == 1.0 and s(799) == 1.0
    assert s(1000) == pytest.approx(0.1)
    x = 0.5
    expect = {"linear": 0.1 + 0.9 * 0.5, "exp": 0.1 ** 0.5, "cosine": 0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * x)),
              "square": 0.1 + 0.9 * (1 - 0.25), "sqrt": 0.1 + 0.9 * (1 - math.sqrt(0.5))}
    expect["miror_cosine"] = 2 * expect["linear"] - expect["cosine"]
    assert s(900) == pytest.approx(expect[kind])
    with pytest.raises(ValueError):
        WSD(10, decay_type="bogus")


def test_powerlaw():
    s = PowerLaw(1000, 10, init_value=1.0, saturation_value=0.2, power=-0.5, time_scale=4.0)
    assert s(5) == pytest.approx(0.5) and s(10) == pytest.approx(1.0)
    assert s(10 + 12) == pytest.approx((1 + 3) ** -0.5)
    assert s(10 ** 6) == pytest.approx(0.2)


def test_scheduler_factory_drives_optimizer_lr():
    from adana_b200.config import flags

    a = flags.defaults()
    a.scheduler, a.iterations, a.warmup_steps, a.lr, a.final_div_factor = "cos_inf", 100, 10, 1e-2, 0.1
    p = torch.nn.Parameter(torch.zeros(2))
    opt = torch.optim.SGD([p], lr=a.lr)
    sch = build_scheduler(a, opt)
    lrs = []
    for _ in range(100):
        lrs.append(opt.param_groups[0]["lr"])
        opt.step()
        sch.step()
    assert lrs[0] == pytest.approx(1e-4) and max(lrs) == pytest.approx(1e-2) and lrs[-1] < 2e-3
    import pickle
    pickle.dumps(sch.state_dict())  # schedules are picklable objects, not closures


def test_schedules_equal_the_reference_functions(ref_src):
    """cos_inf, every WSD decay type and the power-law schedule against the reference's lambdas at every step
    (two steps past the end included)."""
    import importlib.util

    from adana_b200.optim import schedule as mine

    spec = importlib.util.spec_from_file_location("ref_schedule", ref_src / "optim" / "schedule.py")
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)

    def same(f, g, n):
        for t in range(n + 2):
            a, b = f(t), g(t)
            assert abs(a - b) <= 1e-12 * max(1.0, abs(b)), (t, a, b)

    for n, warm, n_inf in ((200, 100, 0), (500, 20, 100), (64, 1, 0)):
        same(mine.cos_inf_schedule(n, warm, 1e2, 1e4, n_inf), ref.cos_inf_schedule(n, warm, 1e2, 1e4, n_inf), n)
    for decay in ("linear", "cosine", "exp", "miror_cosine", "square", "sqrt"):
        for n, warm, frac, final in ((300, 30, 0.1, 0.0), (300, 10, 0.4, 0.05)):
            try:
                g = ref.wsd_schedule(n, final_lr_factor=final, n_warmup=warm, init_div_factor=100, fract_decay=frac, decay_type=decay)
                g(n - 1)
            except Exception:
                continue        # a decay type the reference does not have
            same(mine.wsd_schedule(n, final_lr_factor=final, n_warmup=warm, init_div_factor=100, fract_decay=frac,
                                   decay_type=decay), g, n)
    for power, sat, scale in ((-0.5, 0.0, 1.0), (-1.0, 0.1, 10.0), (-0.25, 0.0, 100.0)):
        same(mine.powerlaw_schedule_with_warmup(400, 40, 1.0, sat, power, scale),
             ref.powerlaw_schedule_with_warmup(400, 40, 1.0, sat, power, scale), 400)


@pytest.mark.parametrize("sched", ["cos_inf", "wsd"])
def test_combined_scheduler_equals_the_reference(ref_src, sched):
    """The Muon scheduler wrapper: same learning rates step by step and the same `state_dict()` keys (one entry per
    parameter group) as the reference's CombinedScheduler."""
    import importlib
    import sys
    import types
    import warnings

    from adana_b200.config import flags
    from adana_b200.optim import muon as mine

    torch.compiler.set_stance("force_eager")
    if "adana_refoptim" not in sys.modules:
        pkg = types.ModuleType("adana_refoptim")
        pkg.__path__ = [str(ref_src / "optim")]
        sys.modules["adana_refoptim"] = pkg
    ref = importlib.import_module("adana_refoptim.muon")
    cfg = flags.defaults()
    cfg.iterations, cfg.warmup_steps, cfg.scheduler, cfg.lr = 50, 5, sched, 0.02
    out = []
    for mod in (ref, mine):
        ps = [torch.nn.Parameter(torch.randn(8, 4)), torch.nn.Parameter(torch.randn(6))]
        opt = mod.DistributedMuon([{"params": [ps[0]]}, {"params": [ps[1]], "weight_decay": 0.0}], lr=0.02)
        s = mod.CombinedScheduler(opt, cfg)
        lrs = []
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")        # scheduler stepped without an optimizer step
            for _ in range(50):
                s.step()
                lrs.append([g["lr"] for g in opt.param_groups])
        out.append((lrs, sorted(s.state_dict())))
    assert out[0][1] == out[1][1] == ["scheduler_0", "scheduler_1"]
    for a, b in zip(out[0][0], out[1][0]):
        assert a == pytest.approx(b, rel=1e-12)
