"""Optimizer math: against an independent NumPy statement of the update rules, against the
reference's own classes when a copy is installed, and fused flat step vs per-tensor classes."""
import copy
import importlib.util
import sys

import numpy as np
import pytest
import torch

from adana_b200.optim import ADana, AdamWDecayingWD, AdEMAMix, AdEMAMixDecayingWD, DanaStarMK4, newton_schulz5
from adana_b200.optim.muon import DistributedMuon, Manau, Muon
from adana_b200.ops import optim as fused


def numpy_logtime(p, g, m, v, tau, t, lr, lr_peak, delta, kappa, clipsnr, eps, gamma3, wd, wd_decaying, wd_ts):
    """float64 restatement of ADana (tau=None) / Dana-Star."""
    a = delta / (delta + t)
    m = m + a * (g - m)
    v = (1 - a) * v + a * g * g
    den = np.sqrt(v) + eps
    if tau is None:
        n = 1 / den
        af = (1 + t) ** (1 - kappa) * np.abs(m) * n
        if clipsnr is not None:
            af = np.minimum(af, clipsnr)
        upd = -lr * g * n - lr * gamma3 * (np.sign(m) * af + m * n)
    else:
        tau = tau + a * (np.abs(g) / (np.abs(g) + den) - tau)
        ct = np.minimum(tau, 0.5)
        r = np.maximum(ct / (1 - ct), 1 / (1 + t))
        n = np.sqrt(r) / den
        af = np.maximum(tau * t, 1.0) ** (1 - kappa) * np.abs(m) * n / r
        if clipsnr is not None:
            af = np.minimum(af, clipsnr)
        upd = -lr * g * n - lr * gamma3 * np.sign(m) * (r * af + np.abs(m) * n)
    p = p + upd
    sched = lr / lr_peak
    p = p * (1 - wd * sched / (1 + t / wd_ts)) if wd_decaying else p * (1 - wd * sched)
    return p, m, v, tau


@pytest.mark.parametrize("cls,clipsnr", [(ADana, None), (ADana, 2.0), (DanaStarMK4, None), (DanaStarMK4, 2.0)])
def test_logtime_matches_numpy(cls, clipsnr):
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.randn(37, 5, dtype=torch.float64))
    opt = cls([p], lr=3e-3, delta=8.0, kappa=0.85, weight_decay=0.2, clipsnr=clipsnr, wd_decaying=True, wd_ts=4.0,
              gamma_3_factor=0.7)
    pn = p.detach().numpy().copy()
    mn, vn = np.zeros_like(pn), np.zeros_like(pn)
    tn = np.zeros_like(pn) if cls is DanaStarMK4 else None
    for t in range(1, 8):
        lr = 3e-3 * (0.5 + 0.1 * t)
        opt.param_groups[0]["lr"] = lr
        g = torch.randn(37, 5, dtype=torch.float64) * (0.1 if t % 2 else 1e-3)
        p.grad = g.clone()
        opt.step()
        pn, mn, vn, tn = numpy_logtime(pn, g.numpy(), mn, vn, tn, t, lr, 3e-3, 8.0, 0.85, clipsnr, 1e-8, 0.7, 0.2, True, 4.0)
        assert np.allclose(p.detach().numpy(), pn, rtol=1e-9, atol=1e-12)
    st = opt.state[p]
    assert st["step"] == 7 and set(st) >= {"m", "v", "current_alpha", "gradient_norm", "auto_factor_mean", "m_norm"}
    assert ("tau" in st) == (cls is DanaStarMK4)
    assert opt.param_groups[0]["weighted_step_count"] == pytest.approx(sum(0.5 + 0.1 * t for t in range(1, 8)))


def _load_ref(ref_src, rel, name):
    torch.compiler.set_stance("force_eager")
    spec = importlib.util.spec_from_file_location(name, ref_src / rel)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("which", ["adana", "dana-mk4", "dana-star", "dana-star-mk4", "adamw-dwd", "ademamix", "ademamix-dwd"])
def test_matches_reference_classes(ref_src, which):
    torch.manual_seed(1)
    common = dict(lr=2e-3, weight_decay=0.3)
    if which in ("adana", "dana-mk4"):
        R = _load_ref(ref_src, "optim/adana.py", "ref_adana").ADana
        kw = dict(delta=8.0, kappa=0.85, clipsnr=2.0 if which == "dana-mk4" else None, wd_decaying=True, wd_ts=3.0)
        mine, ref = ADana, R
    elif which in ("dana-star", "dana-star-mk4"):
        R = _load_ref(ref_src, "optim/dana_star_mk4.py", "ref_dsmk4").DANA_STAR_MK4
        kw = dict(delta=8.0, kappa=0.85, clipsnr=2.0 if which == "dana-star-mk4" else None, wd_decaying=True, wd_ts=3.0)
        mine, ref = DanaStarMK4, R
    elif which == "adamw-dwd":
        ref = _load_ref(ref_src, "optim/adamw_decaying_wd.py", "ref_adwd").AdamWDecayingWD
        mine, kw = AdamWDecayingWD, dict(betas=(0.9, 0.95), wd_decaying=True, wd_ts=3.0)
    elif which == "ademamix":
        ref = _load_ref(ref_src, "optim/ademamix.py", "ref_adm").AdEMAMix
        mine, kw = AdEMAMix, dict(betas=(0.9, 0.95, 0.999), alpha=3.0, beta3_warmup=20, alpha_warmup=20, gamma_3_factor=0.5)
    else:
        ref = _load_ref(ref_src, "optim/ademamix_decaying_wd.py", "ref_admd").AdEMAMix_DecayingWD
        mine, kw = AdEMAMixDecayingWD, dict(betas=(0.9, 0.95, 0.999), alpha=3.0, beta3_warmup=20, alpha_warmup=20,
                                            wd_decaying=True, wd_ts=3.0)
    w0 = [torch.randn(16, 8), torch.randn(8)]
    pa = [torch.nn.Parameter(w.clone()) for w in w0]
    pb = [torch.nn.Parameter(w.clone()) for w in w0]
    oa, ob = mine(pa, **common, **kw), ref(pb, **common, **kw)
    for t in range(6):
        for g in (oa.param_groups[0], ob.param_groups[0]):
            g["lr"] = 2e-3 * (1 - 0.1 * t)
        for a, b in zip(pa, pb):
            gr = torch.randn_like(a) * 0.05
            a.grad, b.grad = gr.clone(), gr.clone()
        oa.step()
        ob.step()
    for a, b in zip(pa, pb):
        assert torch.allclose(a, b, rtol=2e-6, atol=1e-7)
    sa, sb = oa.state_dict(), ob.state_dict()
    assert set(sa["state"][0]) >= {k for k in sb["state"][0] if torch.is_tensor(sb["state"][0][k]) and sb["state"][0][k].dim() > 0}


@pytest.mark.parametrize("kind,clipsnr", [(fused.KIND_ADANA, 2.0), (fused.KIND_DANA_STAR, 2.0), (fused.KIND_DANA_STAR, None)])
def test_fused_flat_step_equals_per_tensor(kind, clipsnr):
    torch.manual_seed(2)
    shapes = [(12, 7), (30,), (5, 5)]
    params = [torch.nn.Parameter(torch.randn(*s)) for s in shapes]
    cls = ADana if kind == fused.KIND_ADANA else DanaStarMK4
    opt = cls(params, lr=1e-3, delta=8.0, kappa=0.85, weight_decay=0.1, clipsnr=clipsnr, wd_decaying=True, wd_ts=2.0)
    flat = torch.cat([p.detach().flatten() for p in params]).clone()
    m, v, tau = torch.zeros_like(flat), torch.zeros_like(flat), torch.zeros_like(flat)
    for t in range(1, 5):
        grads = [torch.randn(*s) * 0.1 for s in shapes]
        for p, g in zip(params, grads):
            p.grad = g.clone()
        opt.step()
        fused.fused_step(flat, torch.cat([g.flatten() for g in grads]), m, v, tau if kind == fused.KIND_DANA_STAR else None,
                         None, kind=kind, lr=1e-3, alpha=8 / (8 + t), step=t, kappa=0.85, clipsnr=clipsnr, eps=1e-8,
                         gamma3=1.0, wd_factor=1 - 0.1 / (1 + t / 2.0))
    assert torch.allclose(flat, torch.cat([p.detach().flatten() for p in params]), rtol=1e-6, atol=1e-7)


def test_newton_schulz_orthogonalises():
    torch.manual_seed(3)
    for shape in [(64, 64), (48, 96), (96, 48)]:
        G = torch.randn(*shape)
        X = newton_schulz5(G, steps=5)
        assert X.shape == G.shape
        s = torch.linalg.svdvals(X.float())
        # singular values are pushed into a band around 1 (the smallest ones of a square Gaussian
        # matrix start near 0 and need more than 5 steps)
        assert s.max() < 1.3 and s.median() > 0.6 and (s > 0.5).float().mean() > 0.9
        U, _, Vh = torch.linalg.svd(G, full_matrices=False)
        assert torch.nn.functional.cosine_similarity((U @ Vh).flatten(), X.flatten(), dim=0) > 0.85


def test_muon_family_steps_reduce_a_quadratic():
    torch.manual_seed(4)
    target = torch.randn(32, 16)

    def run(make):
        w = torch.nn.Parameter(torch.zeros(32, 16))
        b = torch.nn.Parameter(torch.zeros(16))
        opt = make(w, b)
        first = None
        for _ in range(40):
            loss = ((w - target) ** 2).sum() + ((b - 1.0) ** 2).sum()
            first = first or loss.item()
            opt.zero_grad() if hasattr(opt, "zero_grad") else None
            w.grad, b.grad = None, None
            loss.backward()
            opt.step()
        return first, loss.item()

    f, l = run(lambda w, b: DistributedMuon([{"params": [w, b]}], lr=0.05, weight_decay=0.0, adamw_betas=(0.9, 0.95)))
    assert l < 0.5 * f
    f, l = run(lambda w, b: Muon([w, b], lr=0.05, adamw_lr=0.05, ns_steps=5))
    assert l < 0.5 * f
    f, l = run(lambda w, b: Manau([{"params": [w, b], "param_names": ["h.0.mlp.c_fc.weight", "ln_f.weight"]}], lr=0.05,
                                  weight_decay=0.0, kappa=0.85, clipsnr=2.0))
    assert l < 0.5 * f
    with pytest.raises(ValueError):
        Manau([{"params": [torch.nn.Parameter(torch.zeros(2, 2))]}])


@pytest.mark.parametrize("shape", [(32, 16), (16, 32), (24, 24)])
def test_newton_schulz_equals_the_reference_iteration(ref_src, shape):
    """The quintic Newton-Schulz iteration against the reference's function on the same fp32 matrix (tall matrices
    are iterated transposed on both sides)."""
    import sys
    import types

    torch.compiler.set_stance("force_eager")
    if "adana_refoptim" not in sys.modules:
        pkg = types.ModuleType("adana_refoptim")
        pkg.__path__ = [str(ref_src / "optim")]
        sys.modules["adana_refoptim"] = pkg
    ref = importlib.import_module("adana_refoptim.muon").zeropower_via_newtonschulz5
    from adana_b200.optim.muon import newton_schulz5

    torch.manual_seed(0)
    G = torch.randn(*shape)
    assert torch.allclose(newton_schulz5(G.clone(), 5).float(), ref(G.clone(), 5).float(), atol=5e-6, rtol=0)


@pytest.mark.parametrize("which", ["dana-mk4", "dana-star-mk4"])
def test_optimizer_state_dicts_are_interchangeable_with_the_reference(ref_src, which):
    """Four steps with one implementation, `state_dict()` loaded into the other, four more steps: the reference's
    checkpoints resume here and the other way round (same keys in `state` and `param_groups`, same trajectories)."""
    import copy

    if which == "dana-mk4":
        ref_cls, mine = _load_ref(ref_src, "optim/adana.py", "ref_adana_sd").ADana, ADana
    else:
        ref_cls, mine = _load_ref(ref_src, "optim/dana_star_mk4.py", "ref_dsmk4_sd").DANA_STAR_MK4, DanaStarMK4
    torch.manual_seed(0)
    w0 = [torch.randn(16, 8), torch.randn(8)]
    grads = [[torch.randn_like(w) * 0.05 for w in w0] for _ in range(8)]

    def make(cls):
        ps = [torch.nn.Parameter(w.clone()) for w in w0]
        return ps, cls(ps, lr=2e-3, weight_decay=0.3, delta=8.0, kappa=0.85, wd_decaying=True, wd_ts=3.0, clipsnr=2.0)

    def run(ps, opt, steps):
        for t in steps:
            for p, g in zip(ps, grads[t]):
                p.grad = g.clone()
            opt.step()

    for first, second in ((ref_cls, mine), (mine, ref_cls)):
        p1, o1 = make(first)
        run(p1, o1, range(4))
        sd = copy.deepcopy(o1.state_dict())
        p2, o2 = make(second)
        assert set(sd["param_groups"][0]) == set(o2.state_dict()["param_groups"][0])
        o2.load_state_dict(sd)
        for a, b in zip(p2, p1):
            a.data.copy_(b.data)
        run(p1, o1, range(4, 8))
        run(p2, o2, range(4, 8))
        assert set(o1.state_dict()["state"][0]) == set(o2.state_dict()["state"][0])
        for a, b in zip(p1, p2):
            assert torch.allclose(a, b, rtol=0, atol=5e-7)
