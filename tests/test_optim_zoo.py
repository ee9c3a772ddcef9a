"""Every `--opt` name builds and makes progress on a small least-squares problem."""
import copy

import pytest
import torch

from adana_b200.config import flags
from adana_b200.optim.registry import build_optimizer

LR = {"sgd": 0.05, "lion": 0.01, "signsgd": 0.01, "signum": 0.01, "adafactor": 0.05, "prodigy": 1.0, "sophiag": 0.05,
      "soap": 0.05, "muon": 0.05, "d-muon": 0.05, "manau": 0.05, "sf-sgd": 0.2, "lamb": 0.05, "mars": 0.05}


@pytest.mark.parametrize("name", flags.OPTIMIZERS)
def test_optimizer_reduces_loss(name):
    torch.manual_seed(0)
    a = flags.defaults()
    a.opt, a.device, a.iterations, a.warmup_steps = name, "cpu", 60, 5
    a.lr = LR.get(name, 0.02)
    a.mars_lr = a.lr
    a.kappa, a.clipsnr, a.weight_decay, a.wd_ts = 0.85, 2.0, 0.0, 10.0
    a.adema_beta3, a.adema_alpha = 0.999, 2.0
    a.momentum, a.nesterov = 0.9, True
    a.muon_lr_factor = 0.05
    model = torch.nn.Sequential(torch.nn.Linear(16, 32, bias=False), torch.nn.Tanh(), torch.nn.Linear(32, 4, bias=False))
    named = dict(model.named_parameters())
    specs = [{"params": [named["0.weight"], named["2.weight"]], "param_names": ["h.0.mlp.c_fc.weight", "h.0.mlp.c_proj.weight"]}]
    opt = build_optimizer(a, model, copy.copy(specs))
    x, y = torch.randn(256, 16), torch.randn(256, 4)
    hooks = {"train": getattr(opt, "train", None)}
    first = last = None
    for it in range(60):
        if name.startswith("sf-"):
            opt.train()
        loss = ((model(x) - y) ** 2).mean()
        first = first if first is not None else loss.item()
        for p in model.parameters():
            p.grad = None
        loss.backward()
        if name == "sophiag":
            if it % 5 == 0:
                opt.update_hessian()
            opt.step(bs=256)
        else:
            opt.step()
        if name == "mars":
            opt.update_last_grad()
    if name.startswith("sf-"):
        opt.eval()
    last = ((model(x) - y) ** 2).mean().item()
    assert last == last and last < first, (name, first, last)
