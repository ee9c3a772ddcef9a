"""The kernel engine on a GPU against the PyTorch fp32 path of the same model."""
import copy

import pytest
import torch

from conftest import tiny_args

pytestmark = pytest.mark.gpu


def _models(name, **kw):
    from adana_b200.models.utils import get_model

    base = dict(n_embd=256, n_head=4, mlp_hidden_dim=512, sequence_length=128, vocab_size=1024)
    base.update(kw)
    a = tiny_args(name, **base)
    torch.manual_seed(0)
    ref = get_model(a)
    eng_model = copy.deepcopy(ref).cuda()
    return a, ref, eng_model


@pytest.mark.parametrize("name,kw", [("enoki", {}), ("qwen3", dict(elementwise_attn_output_gate=True, n_kv_head=2)),
                                       ("qwen3", dict(normalization_layer_type="layernorm", qkv_dim=128, n_head=2)),
                                       ("llama", dict(multiple_of=64))])
def test_engine_grads_match_fp32_reference(name, kw):
    from adana_b200.ops import _lib
    from adana_b200.runtime.engine import attach

    a, ref, m = _models(name, **kw)
    a_gpu = copy.copy(a)
    a_gpu.dtype, a_gpu.device = "bfloat16", "cuda:0"
    eng = attach(m, a_gpu, device="cuda:0")
    idx = torch.randint(0, a.vocab_size, (4, 128))
    tgt = torch.randint(0, a.vocab_size, (4, 128))
    out_ref = ref(idx, targets=tgt, compute_accuracy=True)
    out_ref["loss"].backward()
    m.train()
    out = m(idx.cuda(), targets=tgt.cuda(), compute_accuracy=True)
    out["loss"].backward()
    torch.cuda.synchronize()
    _lib.check_status()
    assert abs(out["loss"].item() - out_ref["loss"].item()) < 3e-2
    ref_g = {n: p.grad for n, p in ref.named_parameters()}
    for n, p in m.named_parameters():
        g, r = p.grad.float().cpu(), ref_g[n]
        cos = torch.nn.functional.cosine_similarity(g.flatten(), r.flatten(), dim=0).item()
        assert cos > 0.99, (n, cos)
        assert abs(g.norm().item() - r.norm().item()) / (r.norm().item() + 1e-9) < 5e-2, n


def test_engine_training_decreases_loss_and_matches_cpu_engine():
    """A few dana-star-mk4 steps on the GPU engine track the fp32 CPU engine."""
    from adana_b200.ops import _lib
    from adana_b200.runtime.engine import EngineOptimizer, attach

    losses = {}
    for dev, dt in (("cpu", "float32"), ("cuda:0", "bfloat16")):
        a, ref, _ = _models("enoki")
        a.dtype, a.device, a.opt = dt, dev, "dana-star-mk4"
        a.kappa, a.clipsnr, a.lr, a.wd_decaying, a.wd_ts, a.weight_decay = 0.85, 2.0, 1e-3, True, 5.0, 0.1
        m = ref.to(dev)
        eng = attach(m, a, device=dev)
        specs = m.get_parameter_group_specs()
        for g in specs:
            g["param_names"] = g["params"]
        opt = EngineOptimizer(eng, a.opt, a, specs)
        m.train()
        gen = torch.Generator().manual_seed(1)
        ls = []
        for _ in range(8):
            idx = torch.randint(0, a.vocab_size, (4, 128), generator=gen).to(dev)
            out = m(idx, targets=idx.roll(-1, 1))
            out["loss"].backward()
            eng.grad_norm_and_clip(0.5)
            opt.step()
            opt.zero_grad()
            ls.append(out["loss"].item())
        losses[dev] = ls
    torch.cuda.synchronize()
    _lib.check_status()
    assert losses["cuda:0"][-1] < losses["cuda:0"][0]
    for a_, b_ in zip(losses["cpu"], losses["cuda:0"]):
        assert abs(a_ - b_) / a_ < 2e-2, (losses["cpu"], losses["cuda:0"])


def test_smoke_entry():
    import __graft_entry__ as g

    g.smoke()


def test_gathered_weights_match_resident_weights_on_one_gpu():
    """`--fsdp_weights gathered` on one GPU: the block matrices are read as 128-row-aligned slices through the
    gathering GEMM (forward, GELU, residual and both dgrads); training must follow the resident-weight run."""
    from adana_b200.models.utils import get_model
    from adana_b200.ops.gemm import ShardedWeight
    from adana_b200.runtime.engine import EngineOptimizer, attach

    def run(mode):
        a = tiny_args("enoki", n_embd=512, n_head=8, mlp_hidden_dim=2048, sequence_length=128, vocab_size=1024,
                      opt="dana-star-mk4", kappa=0.85, clipsnr=2.0, lr=2e-3, weight_decay=0.1, wd_decaying=True, wd_ts=3.0,
                      acc_steps=1, dtype="bfloat16", device="cuda:0", fsdp_weights=mode)
        torch.manual_seed(0)
        m = get_model(a).to("cuda:0")
        eng = attach(m, a, device="cuda:0")
        assert isinstance(eng.units[0].W["qkv"], ShardedWeight) == (mode == "gathered")
        specs = m.get_parameter_group_specs()
        for g in specs:
            g["param_names"] = g["params"]
        opt = EngineOptimizer(eng, a.opt, a, specs)
        m.train()
        losses = []
        for step in range(4):
            g = torch.Generator().manual_seed(100 + step)
            idx = torch.randint(0, a.vocab_size, (4, a.sequence_length), generator=g).cuda()
            out = m(idx, targets=idx.roll(-1, 1))
            out["loss"].backward()
            if step == 0:
                grads0 = {k: v.float().clone() for k, v in eng.full_param_dict("grad").items()}
            eng.grad_norm_and_clip(0.5)
            opt.step()
            opt.zero_grad()
            losses.append(out["loss"].item())
        return losses, eng.full_param_dict("master"), grads0

    la, pa, ga = run("resident")
    lb, pb, gb = run("gathered")
    # the first backward, before any optimizer step: the same gradients up to bf16 rounding of the dgrads, whose
    # k-loop starts on another slice
    for k in ga:
        assert ((ga[k] - gb[k]).norm() / (ga[k].norm() + 1e-12)).item() < 1e-2, k
    for x, y in zip(la, lb):
        assert abs(x - y) < 2e-3, (la, lb)
    for k in pa:
        d = (pa[k] - pb[k]).abs()
        # sign-like updates: a different bf16 rounding of one gradient element may flip a step of size ~lr
        assert d.mean().item() < 1.5e-3 and d.max().item() < 3e-2, (k, d.mean().item(), d.max().item())


def test_batch_stager_waits_for_queued_readers_of_a_slot():
    """The host may run ahead of the GPU: a device slot is refilled only after the kernels that were queued on the
    consumer's stream while it was handed out have finished (the copy stream waits for the consumer stream)."""
    from adana_b200.data.readers import PinnedBatchStager

    class Counting:
        local_batch_size, sequence_length = 8, 1024

        def __init__(self):
            self.n = 0

        def sample_batch(self, out=None):
            x, y = out
            x.fill_(self.n)
            y.fill_(self.n + 1000)
            self.n += 1
            return x, y

    for lookahead in (False, True):
        stager = PinnedBatchStager(Counting(), "cuda", depth=2, lookahead=lookahead)
        x0, y0 = stager.next_batch()
        torch.cuda._sleep(400_000_000)           # ~0.2 s of work on the consumer stream "still reading" the slot
        snap_x, snap_y = x0.clone(), y0.clone()   # queued behind the sleep
        for _ in range(3):                       # more batches than slots: slot 0 is refilled
            stager.next_batch()
        torch.cuda.synchronize()
        assert int(snap_x.min()) == 0 and int(snap_x.max()) == 0, lookahead
        assert int(snap_y.min()) == 1000 and int(snap_y.max()) == 1000, lookahead


def test_distributed_muon_kernel_chain_matches_the_torch_path_on_one_gpu():
    """`--opt d-muon` on the GPU engine: momentum, pull + normalise, Newton-Schulz, push and apply as kernels, against the
    same optimizer with the kernel chain switched off (torch ops around the same Newton-Schulz GEMMs)."""
    from adana_b200.ops import _lib
    from adana_b200.parallel.dist_muon import ShardedMuon
    from adana_b200.runtime.engine import attach

    results = {}
    for chain in (True, False):
        a, ref, _ = _models("enoki")
        a.dtype, a.device, a.opt = "bfloat16", "cuda:0", "d-muon"
        a.lr, a.weight_decay, a.momentum, a.nesterov, a.muon_ns_steps, a.beta1, a.beta2 = 2e-3, 0.1, 0.9, True, 5, 0.8, 0.99
        m = ref.to("cuda:0")
        eng = attach(m, a, device="cuda:0", sharded=True)
        specs = m.get_parameter_group_specs()
        for g in specs:
            g["param_names"] = g["params"]
        opt = ShardedMuon(eng, a, specs)
        assert opt.chain is not None
        if not chain:
            opt.chain = None
        init = {k: v.clone() for k, v in eng.full_param_dict("master").items()}
        m.train()
        gen = torch.Generator().manual_seed(3)
        before = _lib.launch_count()
        ls = []
        for _ in range(4):
            idx = torch.randint(0, a.vocab_size, (4, 128), generator=gen).to("cuda:0")
            out = m(idx, targets=idx.roll(-1, 1))
            out["loss"].backward()
            eng.grad_norm_and_clip(0.5)
            opt.step()
            opt.zero_grad()
            ls.append(out["loss"].item())
        torch.cuda.synchronize()
        _lib.check_status()
        results[chain] = (ls, init, eng.full_param_dict("master"), _lib.launch_count() - before,
                          {k: v.clone() for k, v in eng.units[0].state.items()})
    ls_k, init, p_k, _, st_k = results[True]
    ls_t, _, p_t, _, st_t = results[False]
    assert ls_k[-1] < ls_k[0]
    for x, y in zip(ls_k, ls_t):
        assert abs(x - y) / y < 1e-2, (ls_k, ls_t)
    for k in p_t:
        moved = (p_t[k] - init[k]).abs().mean().item()
        diff = (p_k[k] - p_t[k]).abs().mean().item()
        assert moved > 0 and diff < 0.05 * moved, (k, diff, moved)
    for k in ("muon_buffer", "adamw_exp_avg", "adamw_exp_avg_sq"):
        # (the two runs drift apart by rounding from the second step on: compare in norm, not element by element)
        assert ((st_k[k] - st_t[k]).norm() / st_t[k].norm()).item() < 3e-2, k
