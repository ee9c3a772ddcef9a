"""Kernel engine on CPU (every op on its PyTorch reference path): the manual backward against
autograd, gradient accumulation, activation checkpointing, fused optimizer vs per-tensor classes,
checkpoint round trips."""
import copy

import pytest
import torch

from conftest import tiny_args
from adana_b200.models.utils import get_model
from adana_b200.optim import ADana, DanaStarMK4
from adana_b200.runtime.engine import EngineOptimizer, attach

CASES = [("enoki", {}), ("enoki", dict(no_qknorm=True, residual_stream_scalar=0.5, hoyer_loss_coeff=0.01)),
         ("qwen3", dict(elementwise_attn_output_gate=True, n_kv_head=1)),
         ("qwen3", dict(normalization_layer_type="layernorm")), ("llama", dict(multiple_of=32))]


def batch(a, seed=0, B=2):
    g = torch.Generator().manual_seed(seed)
    idx = torch.randint(0, a.vocab_size, (B, a.sequence_length), generator=g)
    tgt = torch.randint(0, a.vocab_size, (B, a.sequence_length), generator=g)
    tgt[0, :3] = -1
    return idx, tgt


@pytest.mark.parametrize("name,kw", CASES)
def test_manual_backward_matches_autograd(name, kw):
    a = tiny_args(name, **kw)
    torch.manual_seed(0)
    ref = get_model(a)
    m = copy.deepcopy(ref)
    idx, tgt = batch(a)
    o_ref = ref(idx, targets=tgt, compute_accuracy=True)
    o_ref["loss"].backward()
    attach(m, a, device="cpu")
    m.train()
    o = m(idx, targets=tgt, compute_accuracy=True)
    o["loss"].backward()
    assert o["loss"].item() == pytest.approx(o_ref["loss"].item(), rel=1e-5)
    assert o["accuracy"].item() == pytest.approx(o_ref["accuracy"].item())
    assert set(o["aux_losses"]) >= set(o_ref["aux_losses"])
    if "z_loss" in o_ref["aux_losses"]:
        assert o["aux_losses"]["z_loss"].item() == pytest.approx(o_ref["aux_losses"]["z_loss"].item(), rel=1e-4)
    ref_g = {n: p.grad for n, p in ref.named_parameters()}
    for n, p in m.named_parameters():
        assert torch.allclose(p.grad, ref_g[n], rtol=1e-3, atol=1e-6), n


def test_grad_accumulation_and_checkpointing_agree():
    a = tiny_args("enoki", acc_steps=2)
    torch.manual_seed(0)
    base = get_model(a)
    grads = {}
    for mode in ("plain", "ckpt"):
        m = copy.deepcopy(base)
        aa = copy.copy(a)
        aa.activation_checkpointing = mode == "ckpt"
        eng = attach(m, aa, device="cpu")
        m.train()
        for micro in range(2):
            idx, tgt = batch(a, seed=micro)
            (m(idx, targets=tgt)["loss"] / 2).backward()
        grads[mode] = {n: p.grad.clone() for n, p in m.named_parameters()}
        assert eng.micro_step == 2
    ref = copy.deepcopy(base)
    for micro in range(2):
        idx, tgt = batch(a, seed=micro)
        (ref(idx, targets=tgt)["loss"] / 2).backward()
    for n, p in ref.named_parameters():
        assert torch.allclose(grads["plain"][n], p.grad, rtol=1e-3, atol=1e-6), n
        assert torch.allclose(grads["ckpt"][n], grads["plain"][n], rtol=1e-5, atol=1e-7), n


@pytest.mark.parametrize("opt_name,cls,clip", [("adana", ADana, None), ("dana-star-mk4", DanaStarMK4, 2.0)])
def test_engine_optimizer_matches_per_tensor_training(opt_name, cls, clip):
    a = tiny_args("enoki", opt=opt_name, kappa=0.85, clipsnr=2.0, lr=2e-3, weight_decay=0.2, wd_decaying=True,
                  wd_ts=3.0, grad_clip=0.5)
    torch.manual_seed(0)
    ref = get_model(a)
    m = copy.deepcopy(ref)
    eng = attach(m, a, device="cpu")
    specs = m.get_parameter_group_specs()
    for g in specs:
        g["param_names"] = g["params"]
    e_opt = EngineOptimizer(eng, opt_name, a, specs)
    named = dict(ref.named_parameters())
    r_specs = ref.get_parameter_group_specs()
    for g in r_specs:
        g["params"] = [named[n] for n in g["params"]]
    r_opt = cls(r_specs, lr=a.lr, delta=8.0, kappa=0.85, weight_decay=0.2, clipsnr=clip, wd_decaying=True, wd_ts=3.0)
    m.train()
    for step in range(4):
        idx, tgt = batch(a, seed=step)
        lr = a.lr * (1 - 0.2 * step)
        for g in list(e_opt.param_groups) + list(r_opt.param_groups):
            g["lr"] = lr
        m(idx, targets=tgt)["loss"].backward()
        gn = eng.grad_norm_and_clip(0.5)
        e_opt.step()
        e_opt.zero_grad()
        ref(idx, targets=tgt)["loss"].backward()
        gn_ref = torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.5)
        r_opt.step()
        r_opt.zero_grad(set_to_none=True)
        assert gn.item() == pytest.approx(gn_ref.item(), rel=1e-4)
    # The update divides by sqrt(v): coordinates whose gradient is ~1e-8 (pure rounding noise of the two
    # summation orders) move by a sizeable fraction of lr in either run, so the comparison is statistical:
    # tiny mean deviation, and no coordinate further apart than a fraction of the total step budget.
    for (n, p), (_, q) in zip(sorted(m.named_parameters()), sorted(ref.named_parameters())):
        d = (p - q).abs()
        assert d.mean().item() < 3e-6 and d.max().item() < 0.1 * 4 * a.lr, (n, d.mean().item(), d.max().item())
    # state dict in the reference layout: decay names first, sorted; per-parameter step/m/v(/tau)
    sd = e_opt.state_dict()
    assert sd["param_groups"][0]["param_names"] == sorted(sd["param_groups"][0]["param_names"])
    assert sd["state"][0]["step"] == 4 and sd["state"][0]["m"].shape == dict(m.named_parameters())[
        sd["param_groups"][0]["param_names"][0]].shape
    rs = r_opt.state_dict()["state"]
    assert torch.allclose(sd["state"][0]["v"], rs[0]["v"], rtol=1e-3, atol=1e-9)
    assert ("tau" in sd["state"][0]) == (cls is DanaStarMK4)


def test_checkpoint_roundtrip_main_pt(tmp_path):
    from adana_b200.train import checkpoint as ck

    a = tiny_args("enoki", opt="dana-star-mk4", kappa=0.85, clipsnr=2.0)
    torch.manual_seed(0)

    def make():
        m = get_model(a)
        eng = attach(m, a, device="cpu")
        specs = m.get_parameter_group_specs()
        for g in specs:
            g["param_names"] = g["params"]
        return m, eng, EngineOptimizer(eng, a.opt, a, specs)

    m, eng, opt = make()
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda s: 1.0 / (1 + s))
    m.train()
    for step in range(3):
        idx, tgt = batch(a, seed=step)
        m(idx, targets=tgt)["loss"].backward()
        eng.grad_norm_and_clip(0.5)
        opt.step()
        sched.step()
    ck.save_checkpoint(m, opt, sched, 3, tmp_path / "latest")
    raw = torch.load(tmp_path / "latest" / "main.pt", weights_only=False)
    assert set(raw) == {"model", "optimizer", "scheduler", "itr"} and raw["itr"] == 3
    assert "transformer.h.0.attn.c_attn.weight" in raw["model"] and "tau" in raw["optimizer"]["state"][0]
    torch.manual_seed(123)
    m2, eng2, opt2 = make()
    sched2 = torch.optim.lr_scheduler.LambdaLR(opt2, lambda s: 1.0 / (1 + s))
    assert ck.load_checkpoint(m2, opt2, sched2, tmp_path / "latest" / "main.pt") == 3
    assert opt2.step_count == 3 and sched2.last_epoch == 3
    for m_ in (m, m2):
        m_.train()
    idx, tgt = batch(a, seed=9)
    outs = []
    for mm, ee, oo in ((m, eng, opt), (m2, eng2, opt2)):
        mm(idx, targets=tgt)["loss"].backward()
        ee.grad_norm_and_clip(0.5)
        oo.step()
        outs.append({n: p.detach().clone() for n, p in mm.named_parameters()})
    for n in outs[0]:
        assert torch.equal(outs[0][n], outs[1][n]), n
    # keys written by a compiled / DDP-wrapped reference run load too
    raw["model"] = {"_orig_mod.module." + k: v for k, v in raw["model"].items()}
    torch.save(raw, tmp_path / "latest" / "main.pt")
    m3, _, opt3 = make()
    ck.load_checkpoint(m3, opt3, None, tmp_path / "latest")
    assert torch.equal(dict(m3.named_parameters())["lm_head.weight"], raw["model"]["_orig_mod.module.lm_head.weight"])


def test_worker_state_roundtrip(tmp_path):
    import random

    import numpy as np

    from adana_b200.data import DataReader, make_zipf_tokens
    from adana_b200.train import checkpoint as ck

    r = DataReader(make_zipf_tokens(20_000, 500), 2, 32, seed=4, auto_shard=False)
    for _ in range(5):
        r.sample_batch()
    ck.save_worker_state(tmp_path, train_reader=r, verbose=False)
    expect = (torch.rand(3), np.random.rand(2), random.random(), r.sample_batch()[0])
    r2 = DataReader(make_zipf_tokens(20_000, 500), 2, 32, seed=4, auto_shard=False)
    torch.rand(10), np.random.rand(10), random.random()
    ck.load_worker_state(tmp_path, train_reader=r2, verbose=False)
    assert torch.equal(torch.rand(3), expect[0]) and np.array_equal(np.random.rand(2), expect[1])
    assert random.random() == expect[2] and torch.equal(r2.sample_batch()[0], expect[3])


@pytest.mark.parametrize("opt_name", ["ademamix", "ademamix-decaying-wd"])
def test_engine_ademamix_matches_per_tensor_class(opt_name):
    """The fused flat AdEMAMix step (fast / slow EMA + Adam second moment, alpha and beta3 warm-ups as host scalars)
    against the per-tensor class, which is itself stepped against the reference's in tests/test_optim.py."""
    from adana_b200.optim.adam_family import AdEMAMix, AdEMAMixDecayingWD

    a = tiny_args("enoki", opt=opt_name, lr=2e-3, weight_decay=0.1, wd_decaying=True, wd_ts=3.0, grad_clip=0.5,
                  beta1=0.9, beta2=0.95, adema_beta3=0.99, adema_alpha=3.0, adema_beta3_warmup=6, adema_alpha_warmup=6,
                  gamma_3_factor=0.7)
    torch.manual_seed(0)
    ref = get_model(a)
    m = copy.deepcopy(ref)
    eng = attach(m, a, device="cpu")
    specs = m.get_parameter_group_specs()
    for g in specs:
        g["param_names"] = g["params"]
    e_opt = EngineOptimizer(eng, opt_name, a, specs)
    named = dict(ref.named_parameters())
    r_specs = ref.get_parameter_group_specs()
    for g in r_specs:
        g["params"] = [named[n] for n in g["params"]]
    kw = dict(lr=a.lr, betas=(0.9, 0.95, 0.99), alpha=3.0, beta3_warmup=6, alpha_warmup=6, weight_decay=0.1,
              gamma_3_factor=0.7)
    r_opt = (AdEMAMixDecayingWD(r_specs, wd_decaying=True, wd_ts=3.0, **kw) if opt_name.endswith("wd")
             else AdEMAMix(r_specs, **kw))
    m.train()
    for step in range(4):
        idx, tgt = batch(a, seed=step)
        lr = a.lr * (1 - 0.2 * step)
        for g in list(e_opt.param_groups) + list(r_opt.param_groups):
            g["lr"] = lr
        m(idx, targets=tgt)["loss"].backward()
        eng.grad_norm_and_clip(0.5)
        e_opt.step()
        e_opt.zero_grad()
        ref(idx, targets=tgt)["loss"].backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.5)
        r_opt.step()
        r_opt.zero_grad(set_to_none=True)
    # (coordinates whose gradient is rounding noise move by up to (1 + alpha) lr per step in either run: statistical bound)
    for (n, p), (_, q) in zip(sorted(m.named_parameters()), sorted(ref.named_parameters())):
        d = (p - q).abs()
        assert d.mean().item() < 3e-6 and d.max().item() < 0.1 * 4 * a.lr * 4, (n, d.mean().item(), d.max().item())
    sd = e_opt.state_dict()
    assert {"exp_avg_fast", "exp_avg_slow", "exp_avg_sq", "step"} <= set(sd["state"][0])
    rs = r_opt.state_dict()["state"]
    assert torch.allclose(sd["state"][0]["exp_avg_slow"], rs[0]["exp_avg_slow"], rtol=1e-3, atol=1e-9)
