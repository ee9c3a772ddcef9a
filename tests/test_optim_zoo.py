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


# ---- the same classes against the reference's own, step for step ---------------------------------------------------
def _ref_class(ref_src, rel, cls_name):
    """Import `rel` of the reference's optim directory as a submodule of a private package (so that its relative
    imports resolve) and return the class."""
    import importlib
    import sys
    import types

    torch.compiler.set_stance("force_eager")
    if "adana_refoptim" not in sys.modules:
        pkg = types.ModuleType("adana_refoptim")
        pkg.__path__ = [str(ref_src / "optim")]
        sys.modules["adana_refoptim"] = pkg
    return getattr(importlib.import_module("adana_refoptim." + rel), cls_name)


ZOO_CASES = [
    ("lion", "Lion", {}, 0.0),
    ("sign", "Signum", {"momentum": 0.9}, 0.0),
    ("sign", "Signum", {"momentum": 0.9, "nesterov": True}, 0.0),
    ("sign", "Signum", {"momentum": 0.0}, 0.0),
    ("adopt", "ADOPT", {}, 0.0),
    ("lamb", "Lamb", {}, 1e-7),
    ("adafactor", "Adafactor", {}, 0.0),
    ("adafactor", "Adafactor", {"beta1": 0.9, "relative_step": False, "scale_parameter": False}, 1e-7),
    ("prodigy", "Prodigy", {}, 0.0),
    ("sophia", "SophiaG", {}, 0.0),
    ("mars", "MARS", {}, 5e-6),
    ("mars", "MARS", {"mars_type": "mars-lion"}, 5e-6),
    ("mars", "MARS", {"optimize_1d": True}, 5e-6),
    ("schedulefree", "AdamWScheduleFree", {"warmup_steps": 3}, 0.0),
    ("schedulefree", "SGDScheduleFree", {"momentum": 0.9}, 0.0),
    ("soap", "SOAP", {}, 5e-6),
]


@pytest.mark.parametrize("rel,cls_name,kw,tol", ZOO_CASES, ids=[f"{c[1]}-{i}" for i, c in enumerate(ZOO_CASES)])
def test_zoo_optimizer_follows_the_reference_class(ref_src, rel, cls_name, kw, tol):
    """Six steps on the same random gradients: the parameters must coincide with those of the reference's class
    (exactly where the arithmetic is the same sequence of operations, to rounding where it is regrouped)."""
    from adana_b200.optim import zoo

    ref_cls, mine = _ref_class(ref_src, rel, cls_name), getattr(zoo, cls_name)
    torch.manual_seed(3)
    w0 = [torch.randn(16, 8), torch.randn(8)]
    pa = [torch.nn.Parameter(w.clone()) for w in w0]
    pb = [torch.nn.Parameter(w.clone()) for w in w0]
    base = dict(lr=1.0 if cls_name == "Prodigy" else 2e-3, weight_decay=0.1)
    oa, ob = mine(pa, **base, **kw), ref_cls(pb, **base, **kw)
    for o in (oa, ob):
        if hasattr(o, "train"):
            o.train()
    for _ in range(6):
        for a, b in zip(pa, pb):
            g = torch.randn_like(a) * 0.05
            a.grad, b.grad = g.clone(), g.clone()
        if cls_name == "SophiaG":
            oa.update_hessian()
            ob.update_hessian()
        oa.step()
        ob.step()
    for a, b in zip(pa, pb):
        assert (a - b).abs().max().item() <= tol, (cls_name, kw, (a - b).abs().max().item())
