"""Every `--opt` name under the sharded engine (two Gloo ranks) against one process on the same global batch: the
reference shards first and then hands the parameters to whichever optimizer was asked for
(src/distributed/fsdp.py:105-116, src/main.py:74-253)."""
import pytest
import torch
import torch.distributed as dist

from test_distributed_cpu import _spawn, _t

NAMES = ["adamw", "sgd", "muon", "d-muon", "manau", "soap", "ademamix", "ademamix-decaying-wd", "lion", "sf-adamw",
         "sf-sgd", "signsgd", "signum", "prodigy", "sophiag", "adopt", "mars", "adafactor", "lamb", "adana", "dana-mk4",
         "dana-star", "dana-star-mk4", "adamw-decaying-wd"]
STEPS = 4


def _args(name):
    from conftest import tiny_args

    a = tiny_args("enoki", opt=name, kappa=0.85, clipsnr=2.0, lr=1e-3, weight_decay=0.1, wd_decaying=True, wd_ts=3.0,
                  acc_steps=1, iterations=STEPS, adema_beta3=0.99, adema_alpha=2.0, adema_beta3_warmup=STEPS,
                  adema_alpha_warmup=STEPS, momentum=0.9, nesterov=True, beta1=0.9, beta2=0.95, grad_clip=0.5,
                  precondition_frequency=2, sophia_bs=4, z_loss_coeff=0.0, muon_lr_factor=0.02)
    return a


def _run(rank, world, name):
    from adana_b200.models.utils import get_model
    from adana_b200.optim.registry import build_optimizer
    from adana_b200.parallel.comm import Comm
    from adana_b200.runtime.engine import attach

    if world > 1 and not dist.is_initialized():
        dist.init_process_group("gloo")
    a = _args(name)
    torch.manual_seed(0)
    m = get_model(a)
    eng = attach(m, a, comm=Comm(), sharded=world > 1, device="cpu")
    specs = m.get_parameter_group_specs()
    by_name = dict(m.named_parameters())
    for g in specs:
        g["param_names"] = list(g["params"])
        g["params"] = [by_name[n] for n in g["param_names"]]
    opt = build_optimizer(a, m, specs, engine=eng)
    own = hasattr(opt, "engine") and not hasattr(opt, "inner")      # the engine's fused step or the sharded Muon chain
    m.train()
    per_rank = 4 // world
    for step in range(STEPS):
        g = torch.Generator().manual_seed(100 + step)
        idx_all = torch.randint(0, a.vocab_size, (4, a.sequence_length), generator=g)
        idx = idx_all[rank * per_rank:(rank + 1) * per_rank]
        out = m(idx, targets=idx.roll(-1, 1))
        out["loss"].backward()
        eng.grad_norm_and_clip(a.grad_clip)
        if not own and world == 1:
            for u in eng.units:               # what the backend does for a per-tensor class on the engine's views
                u.grads.mul_(eng._clip[0])
        if name in ("sf-adamw", "sf-sgd"):
            opt.train()
        if name == "sophiag":
            opt.step(bs=a.sophia_bs * a.sequence_length)
        else:
            opt.step()
        if not own:
            eng.refresh_from_master()
        if name == "mars":
            opt.zero_grad(set_to_none=True)
            opt.update_last_grad()
        opt.zero_grad()
        eng.zero_grad()
    full = eng.full_param_dict("master")
    return {k: v.float() for k, v in full.items()}


def _run_all(rank, world, names):
    """All optimizers in one pair of processes (one interpreter start and one rendezvous instead of twenty-four); a
    failure is recorded under its name so that the others still run."""
    import traceback

    dist.init_process_group("gloo")
    out = {}
    for name in names:
        try:
            out[name] = _run(rank, world, name)
        except Exception:
            out[name] = "ERROR " + traceback.format_exc()[-1500:]
    return out


@pytest.fixture(scope="module")
def two_rank_results():
    return _spawn(_run_all, 2, NAMES)


@pytest.mark.timeout(1200)
@pytest.mark.parametrize("name", NAMES)
def test_every_optimizer_steps_under_the_sharded_engine(name, two_rank_results):
    one = _run(0, 1, name)
    two = {r: two_rank_results[r][name] for r in (0, 1)}
    assert not isinstance(two[0], str) and not isinstance(two[1], str), (two[0], two[1])
    init = None
    for k, v in one.items():
        a, b = _t(two[0][k]), _t(two[1][k])
        assert torch.equal(a, b), (name, k)                      # every rank reassembles the same parameters
        assert torch.isfinite(a).all(), (name, k)
        # one process sees the same four sequences as the two ranks together: the same averaged gradient up to fp32
        # summation order, hence the same trajectory up to rounding (sign-based updates flip on ties: a few elements)
        diff = (a - v).abs()
        if name == "muon":
            # bf16 Newton-Schulz products turn a last-bit difference of the gradient into a visible one of the
            # update: compared in norm
            assert (diff.norm() / (v.norm() + 1e-12)).item() < 2e-2, (name, k, diff.max().item())
            continue
        if name == "soap":
            # eigenvectors of nearly degenerate statistics rotate freely under a last-bit change of the gradient: the
            # two runs stay within the distance one step can move a parameter
            assert diff.mean().item() < 1e-3, (name, k, diff.mean().item())
            continue
        tol = 5e-5 + 1e-3 * v.abs()
        frac_bad = (diff > tol).float().mean().item()
        assert frac_bad < (2e-2 if name in ("lion", "signsgd", "signum") else 1e-3), (name, k, frac_bad,
                                                                                     diff.max().item())
