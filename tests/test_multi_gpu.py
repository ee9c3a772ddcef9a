"""Sharded engine on real peers: the peer-memory plane against the NCCL plane (needs >= 2 GPUs)."""
import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "tests"))

pytestmark = pytest.mark.gpu


def _worker(rank, world, plane, weights="resident", sharded=True, reduce_dtype="bfloat16"):
    import torch.distributed as dist

    from conftest import tiny_args
    from adana_b200.models.utils import get_model
    from adana_b200.ops import _lib
    from adana_b200.parallel.comm import Comm
    from adana_b200.runtime.engine import EngineOptimizer, attach

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    a = tiny_args("enoki", n_embd=256, n_head=4, mlp_hidden_dim=512, sequence_length=128, vocab_size=1024,
                  opt="dana-star-mk4", kappa=0.85, clipsnr=2.0, lr=2e-3, weight_decay=0.1, wd_decaying=True, wd_ts=3.0,
                  acc_steps=2, dtype="bfloat16", device=f"cuda:{rank}", fsdp_comm=plane, fsdp_weights=weights,
                  reduce_dtype=reduce_dtype)
    torch.manual_seed(0)
    m = get_model(a).to(a.device)
    eng = attach(m, a, comm=Comm(), sharded=sharded, device=a.device)
    assert ((eng.plane if sharded else eng.ar_plane) is not None) == (plane == "p2p")
    assert (eng.units[0].weights is None) == (weights == "gathered")
    assert eng.reduce_bf16 == (plane == "p2p" and reduce_dtype == "bfloat16")
    specs = m.get_parameter_group_specs()
    for g in specs:
        g["param_names"] = g["params"]
    opt = EngineOptimizer(eng, a.opt, a, specs)
    m.train()
    losses, norms = [], []
    for step in range(4):
        for micro in range(2):
            g = torch.Generator().manual_seed(1000 * step + 10 * micro + rank)
            idx = torch.randint(0, a.vocab_size, (2, a.sequence_length), generator=g).to(a.device)
            eng.sync_on_backward = micro == 1
            out = m(idx, targets=idx.roll(-1, 1))
            (out["loss"] / 2).backward()
        norms.append(float(eng.grad_norm_and_clip(0.5)))
        opt.step()
        opt.zero_grad()
        losses.append(out["loss"].item())
    torch.cuda.synchronize()
    _lib.check_status()
    full = eng.full_param_dict("master")
    return {"losses": losses, "norms": norms, "params": {k: v.float().cpu() for k, v in full.items()}}


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_p2p_plane_matches_nccl_plane():
    from test_distributed_cpu import _spawn, _t

    world = 2
    res = {plane: _spawn(_worker, world, plane) for plane in ("nccl", "p2p")}
    for r in range(world):
        assert res["p2p"][r]["losses"][-1] < res["p2p"][r]["losses"][0]
    for a, b in zip(res["nccl"][0]["norms"], res["p2p"][0]["norms"]):
        assert abs(a - b) / a < 2e-2
    for k, v in res["nccl"][0]["params"].items():
        d = (_t(res["p2p"][0]["params"][k]) - _t(v)).abs()
        assert d.mean().item() < 2e-4, (k, d.mean().item())
        assert torch.equal(_t(res["p2p"][0]["params"][k]), _t(res["p2p"][1]["params"][k]))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("sharded,reduce_dtype", [(True, "float32"), (False, "bfloat16"), (False, "float32")],
                         ids=["fsdp_fp32_wire", "ddp_all_reduce_bf16_wire", "ddp_all_reduce_fp32_wire"])
def test_flagged_gradient_collectives_match_nccl(sharded, reduce_dtype):
    """The flag-ordered reduce-scatter with an fp32 wire, and the replicated (data-parallel) engine whose gradient
    all-reduce runs on the peer-memory plane, against the same engine on NCCL."""
    from test_distributed_cpu import _spawn, _t

    world = min(4, torch.cuda.device_count())
    res = {plane: _spawn(_worker, world, plane, "resident", sharded, reduce_dtype) for plane in ("nccl", "p2p")}
    for a, b in zip(res["nccl"][0]["norms"], res["p2p"][0]["norms"]):
        assert abs(a - b) / a < 2e-2
    # (a bf16 wire rounds each rank's gradient before the sum: parameters whose gradient is tiny, like the 64 QK-norm
    # weights, may take a normalised step of the other sign in one of the four steps of lr 2e-3)
    tol = 2e-4 if reduce_dtype == "float32" else 1e-3
    for k, v in res["nccl"][0]["params"].items():
        d = (_t(res["p2p"][0]["params"][k]) - _t(v)).abs()
        assert d.mean().item() < tol, (k, d.mean().item())
        for r in range(1, world):
            assert torch.equal(_t(res["p2p"][0]["params"][k]), _t(res["p2p"][r]["params"][k]))


def _gather_gemm_worker(rank, world):
    """All-gather fused into the GEMM over real peers: every rank holds `rps` rows of W in symmetric memory and
    computes the full y = x Wᵀ (and dx = dy W) reading the other shards through peer pointers."""
    import torch.distributed as dist

    from adana_b200.ops import _lib, gemm
    from adana_b200.parallel.p2p import P2PPlane

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    M, K, rps = 2048, 1024, 352
    N = world * rps
    plane = P2PPlane.create((rps + 384) * K * 2 + (1 << 16), torch.device("cuda", rank))
    torch.manual_seed(5)
    w = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()                 # same on every rank
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    dy = (torch.randn(M, N, device="cuda") * 0.5).bfloat16()
    mine = plane.alloc(rps * K, torch.bfloat16).view(rps, K)
    mine.copy_(w[rank * rps:(rank + 1) * rps])
    torch.cuda.synchronize()
    plane.barrier()                                                          # every shard is in place
    ptrs = plane.peer_ptrs(mine)
    y = gemm.linear_fwd_gathered(x, ptrs, rps)
    dx = gemm.linear_dgrad_gathered(dy, ptrs, rps, K)
    # staged variant: slices cut on whole tiles; the remote slices cross the link once into a local staging matrix
    rps2 = 384
    N2 = world * rps2
    w2 = (torch.randn(N2, K, device="cuda") * 0.5).bfloat16()
    dy2 = (torch.randn(M, N2, device="cuda") * 0.5).bfloat16()
    mine2 = plane.alloc(rps2 * K, torch.bfloat16).view(rps2, K)
    mine2.copy_(w2[rank * rps2:(rank + 1) * rps2])
    torch.cuda.synchronize()
    plane.barrier()
    ptrs2 = plane.peer_ptrs(mine2)
    ys = [gemm.linear_fwd_gathered(x, ptrs2, rps2, me=rank, staged=True) for _ in range(3)]
    dxs = gemm.linear_dgrad_gathered(dy2, ptrs2, rps2, K, me=rank, staged=True)
    torch.cuda.synchronize()
    plane.barrier()                                                          # nobody frees a shard still being read
    torch.cuda.synchronize()
    _lib.check_status()
    ref_y, ref_dx = x.float() @ w.float().t(), dy.float() @ w.float()
    err_y = ((y.float() - ref_y).norm() / ref_y.norm()).item()
    err_dx = ((dx.float() - ref_dx).norm() / ref_dx.norm()).item()
    old = gemm.set_mode(3)
    same_bits = all(torch.equal(v, gemm.linear_fwd(x, w2)) for v in ys)
    gemm.set_mode(old)
    ref_dx2 = dy2.float() @ w2.float()
    err_dxs = ((dxs.float() - ref_dx2).norm() / ref_dx2.norm()).item()
    return {"err_y": err_y, "err_dx": err_dx, "staged_same_bits": same_bits, "err_dx_staged": err_dxs}


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_gather_gemm_over_nvlink_peers():
    from test_distributed_cpu import _spawn

    world = min(torch.cuda.device_count(), 8)
    res = _spawn(_gather_gemm_worker, world)
    for r in range(world):
        assert res[r]["err_y"] < 8e-3 and res[r]["err_dx"] < 8e-3, res[r]
        assert res[r]["staged_same_bits"] and res[r]["err_dx_staged"] < 8e-3, res[r]


def _gemm_rs_worker(rank, world):
    """Row-parallel linear fused with its reduce-scatter over real peers (parallel/tensor_parallel.RowParallelLinear):
    every rank multiplies its K-slice and the epilogue adds each row into its owner's buffer over NVLink."""
    import torch.distributed as dist

    from adana_b200.ops import _lib
    from adana_b200.parallel.p2p import P2PPlane
    from adana_b200.parallel.tensor_parallel import RowParallelLinear

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    M, N, Kl = 4096, 2304, 576
    K = world * Kl
    torch.manual_seed(9)
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()                 # same on every rank
    w = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    plane = P2PPlane.create((M // world) * N * 4 + 2 * M * N * 2 + (1 << 16), torch.device("cuda", rank))
    xr, wr = x[:, rank * Kl:(rank + 1) * Kl].contiguous(), w[:, rank * Kl:(rank + 1) * Kl].contiguous()
    errs = []
    for mode in ("push", "atomic", "pull"):
        op = RowParallelLinear(plane, M, N, mode=mode)
        for _ in range(3):                                                   # the buffers are reused call after call
            out = op(xr, wr)
            torch.cuda.synchronize()
            ref = (x.float() @ w.float().t())[rank * op.rows:(rank + 1) * op.rows]
            errs.append(((out - ref).norm() / ref.norm()).item())
            plane.barrier()                                                  # nobody zeroes a buffer still being read
    torch.cuda.synchronize()
    _lib.check_status()
    return {"errs": errs}


def _ep_p2p_worker(rank, world):
    """Expert-parallel MoE with its dispatch / combine exchanges over the peer-memory plane against the local MoE
    holding all experts (forward, input gradient, router gradient), and against the NCCL exchange."""
    import torch.distributed as dist
    from conftest import tiny_args

    from adana_b200.models.moe import MoE
    from adana_b200.models.qwen3 import Qwen3MLP
    from adana_b200.ops import _lib
    from adana_b200.parallel.expert_parallel import ExpertParallelMoE

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    a = tiny_args("qwen3", moe=True, moe_num_experts=4 * world, moe_num_shared_experts=0, moe_num_experts_per_tok=2,
                  moe_expert_capacity_factor=0.0, n_embd=128, mlp_hidden_dim=256)
    torch.manual_seed(0)
    dense = MoE(a, Qwen3MLP).cuda()                  # same weights on every rank
    out = {}
    for comm in ("p2p", "nccl"):
        os.environ["ADANA_EP_COMM"] = comm
        torch.manual_seed(1)
        ep = ExpertParallelMoE(a, Qwen3MLP).cuda()
        with torch.no_grad():
            ep.router.weight.copy_(dense.router.weight)
            for e in range(ep.per_rank):
                ep.experts[e].load_state_dict(dense.experts[rank * ep.per_rank + e].state_dict())
        torch.manual_seed(100 + rank)
        x = torch.randn(4, 64, a.n_embd, device="cuda", requires_grad=True)
        for _ in range(2):                           # the buffers are reused from call to call
            x.grad = None
            ep.zero_grad()
            y, _ = ep(x)
            y.sum().backward()
        g_ep = x.grad.clone()
        x.grad = None
        y_ref, _ = dense(x)
        y_ref.sum().backward()
        torch.cuda.synchronize()
        out[comm] = {"err": (y - y_ref).abs().max().item(), "gerr": (g_ep - x.grad).abs().max().item(),
                     "router_grad": ep.router.weight.grad.abs().sum().item(), "used_p2p": bool(ep._p2p_ok)}
    _lib.check_status()
    return out


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_exchanges_over_peer_memory():
    from test_distributed_cpu import _spawn

    world = min(torch.cuda.device_count(), 8)
    res = _spawn(_ep_p2p_worker, world)
    for r in range(world):
        assert res[r]["p2p"]["used_p2p"] and not res[r]["nccl"]["used_p2p"], res[r]
        for comm in ("p2p", "nccl"):
            assert res[r][comm]["err"] < 1e-4 and res[r][comm]["gerr"] < 1e-4 and res[r][comm]["router_grad"] > 0, res[r]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_gemm_fused_with_reduce_scatter_over_nvlink_peers():
    from test_distributed_cpu import _spawn

    world = min(torch.cuda.device_count(), 8)
    res = _spawn(_gemm_rs_worker, world)
    for r in range(world):
        assert max(res[r]["errs"]) < 6e-3, res[r]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_gathered_weights_over_peers_match_resident_weights():
    """Every rank keeps only its row slices of the block matrices; forward / backward GEMMs fetch the other rows
    from the peers and the optimizer stores each new bf16 value at its owner.  Same result as resident weights."""
    from test_distributed_cpu import _spawn, _t

    world = 2
    res = {w: _spawn(_worker, world, "p2p", w) for w in ("resident", "gathered")}
    for a, b in zip(res["resident"][0]["losses"], res["gathered"][0]["losses"]):
        assert abs(a - b) < 5e-3
    for k, v in res["resident"][0]["params"].items():
        d = (_t(res["gathered"][0]["params"][k]) - _t(v)).abs()
        # (a sign-like update: the few elements whose gradient is next to zero may move by a step in either direction)
        assert d.mean().item() < 2e-4 and (d > 5e-3).float().mean().item() < 1e-3 and d.max().item() < 5e-2, \
            (k, d.mean().item(), d.max().item())
        assert torch.equal(_t(res["gathered"][0]["params"][k]), _t(res["gathered"][1]["params"][k]))


def _muon_worker(rank, world, plane):
    import torch.distributed as dist

    from conftest import tiny_args
    from adana_b200.models.utils import get_model
    from adana_b200.ops import _lib
    from adana_b200.parallel.comm import Comm
    from adana_b200.parallel.dist_muon import ShardedMuon
    from adana_b200.runtime.engine import attach

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    a = tiny_args("qwen3", n_embd=256, n_head=4, n_kv_head=2, mlp_hidden_dim=512, sequence_length=128, vocab_size=1024,
                  opt="d-muon", lr=2e-3, weight_decay=0.1, momentum=0.9, nesterov=True, muon_ns_steps=5, beta1=0.8,
                  beta2=0.99, acc_steps=1, dtype="bfloat16", device=f"cuda:{rank}", fsdp_comm=plane)
    torch.manual_seed(0)
    m = get_model(a).to(a.device)
    eng = attach(m, a, comm=Comm(), sharded=True, device=a.device)
    specs = m.get_parameter_group_specs()
    for g in specs:
        g["param_names"] = g["params"]
    opt = ShardedMuon(eng, a, specs)
    assert (opt.chain is not None) == (plane == "p2p")
    m.train()
    losses = []
    for step in range(4):
        g = torch.Generator().manual_seed(1000 * step + rank)
        idx = torch.randint(0, a.vocab_size, (2, a.sequence_length), generator=g).to(a.device)
        out = m(idx, targets=idx.roll(-1, 1))
        out["loss"].backward()
        eng.grad_norm_and_clip(0.5)
        opt.step()
        opt.zero_grad()
        losses.append(out["loss"].item())
    torch.cuda.synchronize()
    _lib.check_status()
    full = eng.full_param_dict("master")
    w0 = eng.units[0].weights.float().cpu()
    return {"losses": losses, "params": {k: v.float().cpu() for k, v in full.items()}, "w0": w0}


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_distributed_muon_chain_over_peers_matches_the_collective_path():
    """`d-muon` under the sharded engine: owners pull their matrices over NVLink, orthogonalise and push the results to
    the holders (kernel chain) against the all-gather / reduce-scatter fallback over NCCL; both on every GPU here."""
    from test_distributed_cpu import _spawn, _t

    world = min(torch.cuda.device_count(), 4)
    res = {plane: _spawn(_muon_worker, world, plane) for plane in ("nccl", "p2p")}
    for r in range(world):
        assert torch.equal(_t(res["p2p"][r]["w0"]), _t(res["p2p"][0]["w0"]))       # the pushed bf16 weights agree everywhere
    for x, y in zip(res["nccl"][0]["losses"], res["p2p"][0]["losses"]):
        assert abs(x - y) / x < 1e-2
    for k, v in res["nccl"][0]["params"].items():
        d = (_t(res["p2p"][0]["params"][k]) - _t(v)).abs().mean().item()
        assert d < 3e-4, (k, d)


def _tp_worker(rank, world, tp, replicas=1):
    """`replicas` > 1 (single process only): the batches of that many data-parallel replicas as accumulated micro-steps."""
    import torch.distributed as dist

    from conftest import tiny_args
    from adana_b200.models.utils import get_model
    from adana_b200.ops import _lib
    from adana_b200.parallel.comm import Comm
    from adana_b200.runtime.engine import EngineOptimizer, attach

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    tp_group = dp_group = None
    if tp > 1:
        for i in range(world // tp):
            ranks = list(range(i * tp, (i + 1) * tp))
            g = dist.new_group(ranks)
            if rank in ranks:
                tp_group = g
        for j in range(tp):
            ranks = list(range(j, world, tp))
            g = dist.new_group(ranks)
            if rank in ranks:
                dp_group = g
    a = tiny_args("qwen3", n_embd=256, n_head=4, n_kv_head=2, qkv_dim=64, mlp_hidden_dim=512, sequence_length=128,
                  vocab_size=1024, opt="adamw", lr=1e-3, weight_decay=0.1, beta1=0.9, beta2=0.99, acc_steps=1,
                  dtype="bfloat16", device=f"cuda:{rank}")
    torch.manual_seed(0)
    m = get_model(a).to(a.device)
    eng = attach(m, a, comm=Comm(dp_group) if tp > 1 else Comm(), sharded=True, device=a.device, tp_group=tp_group)
    specs = m.get_parameter_group_specs()
    for g in specs:
        g["param_names"] = g["params"]
    opt = EngineOptimizer(eng, a.opt, a, specs)
    m.train()
    losses, norms = [], []
    for step in range(4):
        mine = list(range(replicas)) if replicas > 1 else [rank // tp if tp > 1 else rank]
        for i, rep in enumerate(mine):
            g = torch.Generator().manual_seed(1000 * step + rep)
            idx = torch.randint(0, a.vocab_size, (2, a.sequence_length), generator=g).to(a.device)
            eng.sync_on_backward = i == len(mine) - 1
            eng.loss_scale = 1.0 / len(mine)
            out = m(idx, targets=idx.roll(-1, 1))
            (out["loss"] / len(mine)).backward()
        norms.append(float(eng.grad_norm_and_clip(0.5)))
        opt.step()
        opt.zero_grad()
        losses.append(out["loss"].item())
    torch.cuda.synchronize()
    _lib.check_status()
    full = eng.full_param_dict("master")
    on_plane = eng.tp is not None and eng.tp.plane is not None
    return {"losses": losses, "norms": norms, "params": {k: v.float().cpu() for k, v in full.items()}, "plane": on_plane}


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tensor_parallel_engine_over_peer_memory_matches_one_gpu():
    """`--tp_size 2` on the kernel engine: the partial products of the row-parallel GEMMs and of the column-parallel
    dgrads are summed over NVLink from symmetric buffers; against the same model on one GPU."""
    from test_distributed_cpu import _spawn, _t

    one = _spawn(_tp_worker, 1, 1)[0]
    two = _spawn(_tp_worker, 2, 2)
    assert two[0]["plane"] and two[1]["plane"]
    for r in range(2):
        for x, y in zip(two[r]["losses"], one["losses"]):
            assert abs(x - y) / y < 5e-3, (two[r]["losses"], one["losses"])
        for x, y in zip(two[r]["norms"], one["norms"]):
            assert abs(x - y) / y < 2e-2
        for k, v in one["params"].items():
            got = _t(two[r]["params"][k])
            assert tuple(got.shape) == tuple(_t(v).shape)
            assert (got - _t(v)).abs().mean().item() < 3e-4, k
    for k in one["params"]:            # both tp ranks hold bitwise the same replicated state and assemble the same tensors
        assert torch.equal(_t(two[0]["params"][k]), _t(two[1]["params"][k])), k


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_data_by_tensor_parallel_engine_on_four_gpus_matches_one_gpu():
    """2 data-parallel x 2 tensor-parallel ranks: the flat shards and the gradient reduce-scatter run on a peer-memory plane
    over each data-parallel pair, the tensor-parallel sums on a second plane over each tp pair; against one GPU that
    accumulates the two replicas' batches."""
    from test_distributed_cpu import _spawn, _t

    one = _spawn(_tp_worker, 1, 1, 2)[0]
    four = _spawn(_tp_worker, 4, 2)
    for r in range(4):
        assert four[r]["plane"]
        for x, y in zip(four[r]["norms"], one["norms"]):
            assert abs(x - y) / y < 2e-2, (four[r]["norms"], one["norms"])
        for k, v in one["params"].items():
            got = _t(four[r]["params"][k])
            assert tuple(got.shape) == tuple(_t(v).shape)
            assert (got - _t(v)).abs().mean().item() < 3e-4, k
    for k in one["params"]:
        for r in range(1, 4):
            assert torch.equal(_t(four[0]["params"][k]), _t(four[r]["params"][k])), (k, r)
