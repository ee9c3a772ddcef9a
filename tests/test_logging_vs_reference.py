"""The scalar logging helpers against the reference's functions (src/optim/utils.py:462-640): parameter norms and
the `optimizer/*` schedule metrics that the reference's plotting scripts read."""
import sys
import types

import pytest
import torch

from adana_b200.logging.schedules import get_parameter_norms, log_optimizer_schedules
from adana_b200.optim.adam_family import AdEMAMix
from adana_b200.optim.logtime import ADana, DanaStarMK4


def _ref_utils(ref_src, monkeypatch):
    import importlib.util

    if "wandb" not in sys.modules:
        try:
            import wandb  # noqa: F401
        except Exception:
            monkeypatch.setitem(sys.modules, "wandb", types.ModuleType("wandb"))
    spec = importlib.util.spec_from_file_location("ref_optim_utils", ref_src / "optim" / "utils.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_parameter_norms_equal_the_reference(ref_src, monkeypatch):
    ref = _ref_utils(ref_src, monkeypatch)
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(7, 5), torch.nn.Linear(5, 3, bias=False))
    for order in (2, 1, float("inf")):
        assert get_parameter_norms(model, order) == pytest.approx(ref.get_parameter_norms(model, order), rel=1e-6)


@pytest.mark.parametrize("name", ["adana", "dana-mk4", "dana-star-mk4", "ademamix"])
def test_optimizer_schedule_metrics_equal_the_reference(ref_src, monkeypatch, name):
    ref = _ref_utils(ref_src, monkeypatch)
    torch.manual_seed(1)
    ps = [torch.nn.Parameter(torch.randn(8, 4)), torch.nn.Parameter(torch.randn(6))]
    if name == "ademamix":
        opt = AdEMAMix(ps, lr=1e-3, betas=(0.9, 0.95, 0.999), alpha=3.0, beta3_warmup=20, alpha_warmup=20)
    elif name == "dana-star-mk4":
        opt = DanaStarMK4(ps, lr=1e-3, delta=8.0, kappa=0.85, clipsnr=2.0, weight_decay=0.1, wd_decaying=True, wd_ts=3.0)
    else:
        opt = ADana(ps, lr=1e-3, delta=8.0, kappa=0.85, clipsnr=2.0 if name == "dana-mk4" else None, weight_decay=0.1,
                    wd_decaying=True, wd_ts=3.0)
    for _ in range(4):
        for p in ps:
            p.grad = torch.randn_like(p) * 0.1
        opt.step()
    want = ref.log_optimizer_schedules(opt, name)
    got = log_optimizer_schedules(opt, name)
    assert want and set(got) == set(want)
    for k in want:
        assert got[k] == pytest.approx(want[k], rel=1e-6), k
