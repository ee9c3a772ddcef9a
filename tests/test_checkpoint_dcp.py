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
