"""Checkpoints in the `torch.distributed.checkpoint` layout that the reference writes under FSDP
(src/optim/utils.py:275-298: `dcp.save({"model": ..., "optimizer": ...}, <ckpt>/sharded)` + `meta.pt`) are read here:
full tensors are reassembled without a process group and training continues as if never interrupted."""
import pytest
import torch

from conftest import tiny_args


def _build(engine):
    from adana_b200.models.utils import get_model
    from adana_b200.optim.logtime import DanaStarMK4

    a = tiny_args("enoki")
    torch.manual_seed(0)
    m = get_model(a)
    specs = m.get_parameter_group_specs()
    kw = dict(lr=1e-3, delta=8.0, kappa=0.85, clipsnr=2.0, weight_decay=0.1, wd_decaying=True, wd_ts=5.0)
    if engine:
        from adana_b200.runtime.engine import EngineOptimizer, attach

        for k, v in dict(opt="dana-star-mk4", acc_steps=1, gamma_3_factor=1.0, **kw).items():
            setattr(a, k, v)
        eng = attach(m, a, device="cpu")
        for g in specs:
            g["param_names"] = g["params"]
        return m, EngineOptimizer(eng, "dana-star-mk4", a, specs)
    named = dict(m.named_parameters())
    for g in specs:
        g["params"] = [named[n] for n in g["params"]]
    return m, DanaStarMK4(specs, **kw)


def _step(m, opt, x):
    m(x, targets=x)["loss"].backward()
    opt.step()
    opt.zero_grad()


@pytest.mark.parametrize("engine", [False, True], ids=["autograd", "engine"])
def test_dcp_checkpoint_is_imported_and_training_continues(tmp_path, engine):
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint.state_dict import get_model_state_dict, get_optimizer_state_dict

    from adana_b200.train.checkpoint import import_dcp, load_checkpoint, model_state_dict

    x = torch.randint(0, 512, (2, 32))
    src_model, src_opt = _build(False)            # the writer: plain modules, as the reference's FSDP run would gather them
    for _ in range(2):
        _step(src_model, src_opt, x)
    ckpt = tmp_path / "latest"
    ckpt.mkdir()
    dcp.save({"model": get_model_state_dict(src_model), "optimizer": get_optimizer_state_dict(src_model, src_opt)},
             checkpoint_id=str(ckpt / "sharded"), no_dist=True)
    torch.save({"scheduler": None, "itr": 2}, ckpt / "meta.pt")

    model_sd, opt_sd = import_dcp(ckpt / "sharded")
    assert set(model_sd) == set(src_model.state_dict()) and "state" in opt_sd and "param_groups" in opt_sd
    m, opt = _build(engine)
    assert load_checkpoint(m, opt, None, ckpt / "main.pt") == 2
    for k, v in src_model.state_dict().items():
        assert torch.equal(model_state_dict(m)[k], v), k
    _step(src_model, src_opt, x)
    _step(m, opt, x)
    got = model_state_dict(m)
    for k, v in src_model.state_dict().items():
        assert torch.allclose(got[k], v, atol=1e-6, rtol=1e-5), k


# ---- written here, read the way the reference reads it -------------------------------------------------------------
def _save_then_load_like_the_reference(rank, world, ckpt_dir):
    """Two ranks of the sharded engine write `<ckpt>/sharded`; then every rank does what the reference's loader does
    (src/optim/utils.py:328-337): `dcp.load` into state dictionaries keyed by parameter name whose tensors are DTensors
    sharded on dimension 0 over the ranks, as FSDP2's `get_model_state_dict` / `get_optimizer_state_dict` hand them out."""
    import torch.distributed as dist
    import torch.distributed.checkpoint as dcp
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor

    from adana_b200.models.utils import get_model
    from adana_b200.parallel.comm import Comm
    from adana_b200.runtime.engine import EngineOptimizer, attach
    from adana_b200.train import checkpoint as ck

    dist.init_process_group("gloo")
    a = tiny_args("enoki", opt="dana-star-mk4", kappa=0.85, clipsnr=2.0, lr=2e-3, weight_decay=0.1, wd_decaying=True,
                  wd_ts=3.0)
    torch.manual_seed(0)
    m = get_model(a)
    eng = attach(m, a, comm=Comm(), sharded=True, device="cpu")
    specs = m.get_parameter_group_specs()
    for g in specs:
        g["param_names"] = g["params"]
    opt = EngineOptimizer(eng, a.opt, a, specs)
    m.train()
    for step in range(2):
        x = torch.randint(0, a.vocab_size, (2, a.sequence_length), generator=torch.Generator().manual_seed(10 * step + rank))
        m(x, targets=x.roll(-1, 1))["loss"].backward()
        eng.grad_norm_and_clip(0.5)
        opt.step()
        opt.zero_grad()
    ck.save_checkpoint(m, opt, None, 2, ckpt_dir)
    want = {k: eng.full_param_dict(k) for k in ("master", "m", "v", "tau")}

    mesh = init_device_mesh("cpu", (world,))
    shapes = {s.name: s.shape for u in eng.units for s in u.layout.slots}

    def sharded_zeros(shape):
        return distribute_tensor(torch.zeros(shape), mesh, [Shard(0)])

    model_sd = {n: sharded_zeros(sh) for n, sh in shapes.items()}
    scalars = ("current_alpha", "gradient_norm", "auto_factor_mean", "current_kappa_factor", "m_norm")
    opt_sd = {"state": {n: {"step": 0, "m": sharded_zeros(sh), "v": sharded_zeros(sh), "tau": sharded_zeros(sh),
                            **{k: torch.zeros(()) for k in scalars}} for n, sh in shapes.items()},
              "param_groups": [{"lr": 0.0, "delta": 0.0, "epsilon": 0.0, "weight_decay": 0.0, "weighted_step_count": 0,
                                "params": []} for _ in opt.param_groups]}
    dcp.load({"model": model_sd, "optimizer": opt_sd}, checkpoint_id=str(ckpt_dir / "sharded"))
    worst = 0.0
    for n in shapes:
        worst = max(worst, (model_sd[n].full_tensor() - want["master"][n]).abs().max().item())
        for k in ("m", "v", "tau"):
            worst = max(worst, (opt_sd["state"][n][k].full_tensor() - want[k][n]).abs().max().item())
    groups = opt_sd["param_groups"]
    return {"worst": worst, "step": opt_sd["state"]["lm_head.weight"]["step"], "lr": groups[0]["lr"],
            "wd": [g["weight_decay"] for g in groups], "n_params": [len(g["params"]) for g in groups],
            "nonzero": float(want["tau"]["lm_head.weight"].abs().sum())}


def test_sharded_checkpoint_written_here_loads_into_fsdp_style_dtensor_state(tmp_path):
    from test_distributed_cpu import _spawn

    res = _spawn(_save_then_load_like_the_reference, 2, tmp_path / "latest")
    for r in (0, 1):
        assert res[r]["worst"] == 0.0 and res[r]["step"] == 2 and res[r]["nonzero"] > 0
        assert res[r]["lr"] == pytest.approx(2e-3) and res[r]["wd"] == [0.1, 0.0] and min(res[r]["n_params"]) > 0
    # and without any process group, as full tensors (what the inference tool and `import_dcp` do)
    from adana_b200.train.checkpoint import import_dcp

    model_sd, opt_sd = import_dcp(tmp_path / "latest" / "sharded")
    assert "transformer.h.0.attn.c_attn.weight" in model_sd and opt_sd["state"]["lm_head.weight"]["step"] == 2
