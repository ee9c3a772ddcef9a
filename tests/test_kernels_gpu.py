"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from adana_b200.ops import _lib, attention, gemm, misc, norm, optim, rope

DEV = "cuda"


def rnd(*s, scale=0.5, dtype=torch.bfloat16):
    return (torch.randn(*s, device=DEV) * scale).to(dtype)


def rel_err(a, b):
    """Largest absolute error over the largest reference magnitude (hides relative error of small entries: used
    next to `assert_close`, not instead of it)."""
    a, b = a.float(), b.float()
    return ((a - b).abs().max() / (b.abs().max() + 1e-6)).item()


def assert_close(a, b, rtol=2e-2, atol=None, what=""):
    """Element-wise |a - b| <= atol + rtol * |b| with constants for bf16 outputs of fp32-accumulated sums: rtol a
    few bf16 ulps (2^-8 = 3.9e-3 each), atol a small fraction of the reference's RMS (cancellation in a sum leaves an
    absolute, not a relative, error)."""
    a, b = a.float(), b.float()
    if atol is None:
        atol = 2e-2 * b.pow(2).mean().sqrt().item() + 1e-6
    bad = (a - b).abs() > atol + rtol * b.abs()
    n_bad = int(bad.sum())
    assert n_bad == 0, (f"{what}: {n_bad} of {bad.numel()} elements off; worst |a-b| = "
                        f"{(a - b).abs().max().item():.4g} at |b| = {b.abs().flatten()[(a - b).abs().argmax()].item():.4g}")


@pytest.fixture(autouse=True)
def _status():
    assert _lib.available(), "kernel library must load on a GPU box"
    yield
    torch.cuda.synchronize()
    _lib.check_status()


@pytest.fixture(params=[0, 1, 2, 3], ids=["auto", "single_cta", "cta_pair_streamk", "cta_pair"])
def gemm_mode(request):
    """Every GEMM test runs once per tile policy (per shape / one CTA per tile / cta_group::2 pair per tile
    with and without stream-K for fp32 outputs)."""
    old = gemm.set_mode(request.param)
    yield request.param
    gemm.set_mode(old)


@pytest.mark.parametrize("M,N,K", [(1024, 768, 512), (1000, 520, 328), (256, 2304, 192), (4096, 1024, 2048)])
def test_gemm_fwd_dgrad_wgrad(M, N, K, gemm_mode):
    torch.manual_seed(0)
    x, w, dy = rnd(M, K), rnd(N, K), rnd(M, N)
    assert rel_err(gemm.linear_fwd(x, w), x.float() @ w.float().t()) < 8e-3
    assert rel_err(gemm.linear_dgrad(dy, w), dy.float() @ w.float()) < 8e-3
    ref = dy.float().t() @ x.float()
    dw = gemm.linear_wgrad(dy, x)
    assert rel_err(dw, ref) < 1e-3
    gemm.linear_wgrad(dy, x, out=dw, accumulate=True, alpha=0.5)
    assert rel_err(dw, 1.5 * ref) < 1e-3


@pytest.mark.parametrize("mode", [0, 2], ids=["last_wave_split", "every_tile_split"])
def test_gemm_wgrad_stream_k_partial_tiles(mode):
    """81 pair tiles on 74 pairs.  Per-shape policy: 74 whole tiles, the other 7 split along K over all pairs;
    mode 2: every K loop split.  Partial tiles meet in C through fp32 vector atomics."""
    torch.manual_seed(3)
    M, N, K = 4096, 2304, 2304
    x, dy = rnd(M, K), rnd(M, N)
    ref = dy.float().t() @ x.float()
    old = gemm.set_mode(mode)
    try:
        dw = torch.full((N, K), 7.0, device=DEV)            # overwrite mode must not see old contents
        gemm.linear_wgrad(dy, x, out=dw)
        assert rel_err(dw, ref) < 1e-3
        gemm.linear_wgrad(dy, x, out=dw, accumulate=True, alpha=0.25)
        assert rel_err(dw, 1.25 * ref) < 1e-3
        view = torch.zeros(N, K + 64, device=DEV)[:, :K]    # row pitch larger than the row
        gemm.linear_wgrad(dy, x, out=view)
        assert rel_err(view, ref) < 1e-3
    finally:
        gemm.set_mode(old)


def test_gemm_epilogues(gemm_mode):
    torch.manual_seed(1)
    M, N, K = 1024, 768, 512
    x, w, dy = rnd(M, K), rnd(N, K), rnd(M, N)
    ref = x.float() @ w.float().t()
    z, h = gemm.linear_gelu_fwd(x, w)
    assert rel_err(z, ref) < 8e-3 and rel_err(h, torch.nn.functional.gelu(ref)) < 8e-3
    r = torch.randn(M, N, device=DEV)
    assert rel_err(gemm.linear_resid_fwd(x, w, r, alpha=0.5), r + 0.5 * ref) < 1e-4
    r2 = r.clone()
    gemm.linear_resid_fwd(x, w, r2, alpha=0.5, out=r2)
    assert rel_err(r2, r + 0.5 * ref) < 1e-4
    zz = rnd(M, K)
    zf = zz.float().requires_grad_(True)
    g, = torch.autograd.grad(torch.nn.functional.gelu(zf).sum(), zf)
    assert rel_err(gemm.linear_dgrad_dgelu(dy, w, zz, alpha=0.7), 0.7 * (dy.float() @ w.float()) * g) < 8e-3
    assert rel_err(gemm.linear_fwd_f32(x, w), ref) < 1e-4


def test_gemm_swiglu(gemm_mode):
    torch.manual_seed(2)
    M, H, K = 512, 384, 256
    x, wgu = rnd(M, K), rnd(2 * H, K)
    gu, h = gemm.linear_swiglu_fwd(x, wgu)
    ref = x.float() @ wgu.float().t()
    assert rel_err(gu, ref) < 8e-3
    assert rel_err(h, torch.nn.functional.silu(ref[:, :H]) * ref[:, H:]) < 8e-3
    wd, dyd = rnd(K, H), rnd(M, K)
    dgu = gemm.linear_dgrad_dswiglu(dyd, wd, gu, alpha=0.5)
    dh = 0.5 * (dyd.float() @ wd.float())
    g, u = gu[:, :H].float(), gu[:, H:].float()
    s = torch.sigmoid(g)
    assert rel_err(dgu, torch.cat([dh * u * s * (1 + g * (1 - s)), dh * g * s], 1)) < 8e-3


@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("cols", [192, 2304, 1000])
def test_norm_fwd_bwd(kind, cols):
    torch.manual_seed(3)
    rows = 777
    x = torch.randn(rows, cols, device=DEV) * 2 + 0.3
    w = torch.rand(cols, device=DEV) + 0.5
    y, mean, rstd = norm.norm_fwd(x, w, 1e-5, kind, torch.bfloat16)
    yr, mr, rr = norm.norm_fwd_ref(x, w, 1e-5, kind, torch.float32)
    assert rel_err(y, yr) < 8e-3 and rel_err(rstd, rr) < 1e-5
    dy = rnd(rows, cols)
    acc = torch.randn(rows, cols, device=DEV)
    acc_ref = acc.clone()
    lp = torch.empty(rows, cols, device=DEV, dtype=torch.bfloat16)
    dx, dw = norm.norm_bwd(dy, x, w, mean, rstd, kind, dx_accum=acc, dx_lowp=lp)
    dxr, dwr = norm.norm_bwd_ref(dy, x, w, mr, rr, kind, dx_accum=acc_ref)
    assert rel_err(dx, dxr) < 1e-4 and rel_err(dw, dwr) < 1e-3 and rel_err(lp, dxr) < 8e-3


@pytest.mark.parametrize("hd,kind,gate", [(64, 0, False), (128, 1, True), (64, 2, False)])
def test_qknorm_rope(hd, kind, gate):
    torch.manual_seed(4)
    B, S, Hq, Hk = 2, 96, 4, 2
    T = B * S
    qs = 2 * hd if gate else hd
    width = Hq * qs + 2 * Hk * hd
    qkv = rnd(T, width, scale=1.0)
    wq, wk = torch.rand(hd, device=DEV) + 0.5, torch.rand(hd, device=DEV) + 0.5
    freqs = rope.precompute_freqs_cis(hd, S).to(DEV)
    args = (0, qs, Hq * qs, hd, wq, wk, freqs, S, Hq, Hk, hd, 1e-5, kind)
    q, k = rope.qknorm_rope_fwd(qkv, *args)
    qr, kr = rope.qknorm_rope_fwd_ref(qkv.float(), *args)
    assert rel_err(q, qr) < 1e-2 and rel_err(k, kr) < 1e-2
    dq, dk = rnd(T, Hq, hd), rnd(T, Hk, hd)
    dqkv = torch.zeros_like(qkv)
    dwq, dwk = rope.qknorm_rope_bwd(dq, dk, qkv, dqkv, *args)
    dref = torch.zeros(T, width, device=DEV)
    dwq_r, dwk_r = rope.qknorm_rope_bwd_ref(dq.float(), dk.float(), qkv.float(), dref, *args)
    assert rel_err(dqkv, dref) < 1e-2
    if kind != 2:
        assert rel_err(dwq, dwq_r) < 5e-3 and rel_err(dwk, dwk_r) < 5e-3
    # the query gradient may arrive in fp32 (the attention backward's accumulator): same values, same result
    dqkv32 = torch.zeros_like(qkv)
    dwq32, dwk32 = rope.qknorm_rope_bwd(dq.float(), dk, qkv, dqkv32, *args)
    assert torch.equal(dqkv32, dqkv)
    if kind != 2:
        assert torch.equal(dwq32, dwq) and torch.equal(dwk32, dwk)


def test_embedding():
    torch.manual_seed(5)
    V, d, T = 1000, 192, 5000
    table = torch.randn(V, d, device=DEV)
    idx = torch.randint(0, V, (T,), device=DEV)
    idx[:100] = 7  # collisions
    assert torch.equal(misc.embedding_fwd(idx, table), table[idx])
    tb = table.to(torch.bfloat16)
    assert torch.equal(misc.embedding_fwd(idx, tb), tb[idx].float())
    dout = torch.randn(T, d, device=DEV)
    dt = torch.zeros(V, d, device=DEV)
    misc.embedding_bwd(idx, dout, dt)
    ref = torch.zeros(V, d, device=DEV).index_add_(0, idx, dout)
    assert rel_err(dt, ref) < 1e-5


@pytest.mark.parametrize("logits_dtype", [torch.bfloat16, torch.float32], ids=["bf16_in_place", "fp32"])
@pytest.mark.parametrize("V,d,T", [(50304, 192, 700), (512, 128, 700), (50304, 256, 16384)])
def test_linear_ce(V, d, T, logits_dtype):
    """fp32 logits, and bf16 logits turned into dlogits in place; the last case has the flagship's row count
    (8 sequences of 2048 tokens, four chunks of 4096 rows)."""
    torch.manual_seed(6)
    h = rnd(T, d, scale=1.0)
    w = rnd(V, d, scale=0.05)
    tgt = torch.randint(0, V, (T,), device=DEV)
    tgt[:5] = -1
    out = misc.linear_ce(h, w, tgt, z_coeff=1e-2, loss_scale=0.5, chunk_rows=256 if T < 4096 else 4096,
                         logits_dtype=logits_dtype)
    ref = misc.linear_ce_ref(h, w, tgt, 1e-2, 0.5)
    for k in ("ce_sum", "z_sum", "valid"):
        assert abs(out[k].item() - ref[k].item()) / (abs(ref[k].item()) + 1e-6) < 2e-3, k
    # bf16 logits can tie where fp32 ones do not: a few argmax flips among T rows
    assert abs(out["correct"].item() - ref["correct"].item()) <= (2 if logits_dtype == torch.float32 else 2 + T // 500)
    assert rel_err(out["dh"], ref["dh"]) < 2e-2
    assert rel_err(out["dw"], ref["dw"]) < 2e-2
    assert_close(out["dh"], ref["dh"], what="dh")
    assert_close(out["dw"], ref["dw"], what="dw")


@pytest.mark.parametrize("kind,clipsnr", [(0, None), (0, 2.0), (1, None), (1, 2.0), (2, None), (3, None), (4, None),
                                          (5, None)])
def test_fused_optimizer(kind, clipsnr):
    """The fused flat step on the GPU against the same step through its PyTorch formulation on the CPU (which the CPU
    tests pin to the per-tensor classes, and those to the reference's own classes): ADana, Dana-Star, AdamW with
    coupled / independent decay, AdEMAMix with coupled / independent decay."""
    torch.manual_seed(7)
    n = 100_003
    mk = lambda: (torch.randn(n, device=DEV), torch.randn(n, device=DEV) * 1e-2,
                  torch.randn(n, device=DEV) * 1e-3, torch.rand(n, device=DEV) * 1e-4, torch.rand(n, device=DEV) * 0.6)
    p, g, m, v, tau = mk()
    cpu = [t.cpu().clone() for t in (p, g, m, v, tau)]
    p16 = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    clip = torch.tensor([0.7, 0.0], device=DEV)
    kw = dict(kind=kind, lr=3e-3, alpha=8 / 15, step=7, kappa=0.85, clipsnr=clipsnr, eps=1e-8, gamma3=1.0,
              wd_factor=0.999, grad_scale=0.5, betas=(0.9, 0.95), beta3=0.97, wd_coupled=0.05)
    diag = torch.zeros(4, device=DEV)
    optim.fused_step(p, g, m, v, tau, p16, clip_coef_t=clip, diag=diag, **kw)
    pc, gc, mc, vc, tc = cpu
    dc = torch.zeros(4)
    optim.fused_step(pc, gc, mc, vc, tc, None, clip_coef_t=clip.cpu(), diag=dc, **kw)
    assert rel_err(p.cpu(), pc) < 1e-5 and rel_err(m.cpu(), mc) < 1e-5 and rel_err(v.cpu(), vc) < 1e-5
    if kind in (1, 4, 5):
        assert rel_err(tau.cpu(), tc) < 1e-5
    assert rel_err(p16.cpu(), pc) < 8e-3
    if kind in (0, 1):
        assert rel_err(diag.cpu(), dc) < 1e-3


def test_sumsq_and_clip():
    x = torch.randn(1_000_001, device=DEV)
    out = torch.zeros(1, device=DEV)
    optim.sumsq_accumulate(x, out)
    assert abs(out.item() - x.double().pow(2).sum().item()) / out.item() < 1e-4
    c = torch.zeros(2, device=DEV)
    optim.clip_coef(out, 0.5, 1.0, c)
    norm_ = math.sqrt(out.item()) * 0.5
    assert abs(c[1].item() - norm_) / norm_ < 1e-5 and abs(c[0].item() - min(1.0, 1.0 / (norm_ + 1e-6))) < 1e-6


def test_sigmoid_gate():
    torch.manual_seed(8)
    T, H, hd = 300, 4, 64
    proj = rnd(T, H * 2 * hd + 128, scale=1.0)
    a = rnd(T, H * hd)
    out = misc.sigmoid_gate_fwd(a, proj, hd, 2 * hd, H, hd)
    g = torch.as_strided(proj, (T, H, hd), (proj.stride(0), 2 * hd, 1), hd).float()
    assert rel_err(out, (a.float().view(T, H, hd) * torch.sigmoid(g)).view(T, -1)) < 8e-3
    dout = rnd(T, H * hd)
    dproj = torch.zeros_like(proj)
    da = misc.sigmoid_gate_bwd(dout, a, proj, dproj, hd, 2 * hd, H, hd)
    s = torch.sigmoid(g)
    assert rel_err(da, (dout.float().view(T, H, hd) * s).view(T, -1)) < 8e-3
    dg = torch.as_strided(dproj, (T, H, hd), (dproj.stride(0), 2 * hd, 1), hd).float()
    assert rel_err(dg, dout.float().view(T, H, hd) * a.float().view(T, H, hd) * s * (1 - s)) < 1e-2


@pytest.mark.parametrize("hd,Hq,Hk,S", [(64, 4, 4, 256), (64, 4, 2, 512), (128, 2, 2, 256), (128, 4, 1, 384)])
def test_attention_forward_native(hd, Hq, Hk, S):
    from adana_b200.ops import attention_native

    torch.manual_seed(9)
    B = 2
    T = B * S
    q, k = rnd(T, Hq, hd, scale=1.0), rnd(T, Hk, hd, scale=1.0)
    width = 3 * Hk * hd + 64
    buf = rnd(T, width, scale=1.0)
    v_off = 64 + Hk * hd
    v = torch.as_strided(buf, (T, Hk, hd), (width, hd, 1), v_off)
    scale = 1.0 / math.sqrt(hd)
    out, lse2 = attention_native.fwd(q, k, buf, v_off, hd, B, S, scale)
    ref, lse = attention.attention_ref(q, k, v, B, S, scale)
    assert rel_err(out, ref) < 2e-2
    assert rel_err(lse2 * math.log(2.0), lse) < 1e-3


@pytest.mark.parametrize("hd,Hq,Hk,S,B", [(64, 4, 4, 256, 2), (64, 4, 2, 512, 2), (128, 2, 2, 256, 2), (128, 4, 1, 384, 2),
                                          (64, 36, 36, 2048, 1), (64, 2, 2, 8192, 1), (128, 16, 8, 4096, 1),
                                          (128, 2, 1, 8192, 1)],
                         ids=["hd64", "hd64_gqa", "hd128", "hd128_mqa", "flagship_36x64x2048", "hd64_S8192",
                              "qwen3_16q8kv_S4096", "hd128_S8192"])
def test_attention_backward_native(hd, Hq, Hk, S, B):
    """Forward + backward; the long cases are the flagship's shape (36 heads of 64 at S = 2048), the Qwen3
    configuration's (16 query / 8 KV heads of 128 at S = 4096) and the longest sequence of the sweep (8192)."""
    from adana_b200.ops import attention_native

    torch.manual_seed(10)
    T = B * S
    q, k = rnd(T, Hq, hd, scale=1.0), rnd(T, Hk, hd, scale=1.0)
    width = 3 * Hk * hd + 64
    buf = rnd(T, width, scale=1.0)
    v_off = 64 + Hk * hd
    v = torch.as_strided(buf, (T, Hk, hd), (width, hd, 1), v_off)
    scale = 1.0 / math.sqrt(hd)
    out, lse2 = attention_native.fwd(q, k, buf, v_off, hd, B, S, scale)
    dout = rnd(T, Hq * hd, scale=1.0)
    dbuf = torch.zeros_like(buf)
    dq, dk = attention_native.bwd(dout, q, k, buf, v_off, hd, B, S, scale, lse2, out, dbuf)
    qd, kd, vd = (t.float().detach().requires_grad_(True) for t in (q, k, v))
    ref, _ = attention.attention_ref(qd, kd, vd, B, S, scale)
    rq, rk, rv = torch.autograd.grad(ref, (qd, kd, vd), dout.float())
    dv = torch.as_strided(dbuf, (T, Hk, hd), (width, hd, 1), v_off)
    assert rel_err(dq, rq) < 3e-2, "dq"
    assert rel_err(dk, rk) < 3e-2, "dk"
    assert rel_err(dv, rv) < 3e-2, "dv"
    assert rel_err(out, ref) < 2e-2, "out"
    # element-wise as well: P and dS are rounded to bf16 before the products, so the absolute term is a few percent
    # of the gradient's RMS
    for got, want, name in ((dq, rq, "dq"), (dk, rk, "dk"), (dv, rv, "dv")):
        assert_close(got, want, rtol=3e-2, atol=1e-1 * want.float().pow(2).mean().sqrt().item(), what=name)
    untouched = dbuf.clone()
    untouched.as_strided((T, Hk, hd), (width, hd, 1), v_off).zero_()
    assert untouched.abs().max().item() == 0.0


# ---- peer-memory collectives in fake-peer mode: every "rank" is an allocation on this one GPU ----------
def test_p2p_reduce_scatter_and_clip_fake_peers():
    from adana_b200.parallel.p2p import P2PPlane

    torch.manual_seed(11)
    world, n = 4, 64 * 4 * 257
    planes = P2PPlane.fake(n * 4 + 4096, world, DEV)
    grads = [pl.alloc(n, torch.float32) for pl in planes]
    for g in grads:
        g.copy_(torch.randn(n, device=DEV))
    total = torch.stack(grads).sum(0)
    shard = n // world
    partial = []
    for r, pl in enumerate(planes):
        out = torch.empty(shard, device=DEV)
        ss = torch.zeros(1, device=DEV)
        pl.reduce_scatter_sumsq(grads[r], r * shard, out, ss)
        assert rel_err(out, total[r * shard:(r + 1) * shard]) < 1e-6
        assert abs(ss.item() - out.double().pow(2).sum().item()) / ss.item() < 1e-4
        partial.append(ss)
    # every rank publishes its partial into every arena; the flag barrier itself is exercised on real peers
    lib = _lib.lib()
    for r, pl in enumerate(planes):
        _lib.check_rc(lib.adana_p2p_publish_f32(pl._slot_ptrs, r, world, partial[r].data_ptr(), _lib.stream_ptr()), "publish")
    out = torch.zeros(2, device=DEV)
    _lib.check_rc(lib.adana_clip_coef_multi(planes[2].slots.data_ptr(), world, 1.0 / world, 1.0, out.data_ptr(),
                                            _lib.stream_ptr()), "clip")
    norm = total.double().norm().item() / world
    assert abs(out[1].item() - norm) / norm < 1e-4 and abs(out[0].item() - min(1.0, 1.0 / (norm + 1e-6))) < 1e-5


@pytest.mark.parametrize("kind", [0, 1, 2])
def test_p2p_opt_step_push_fake_peers(kind):
    from adana_b200.parallel.p2p import P2PPlane

    torch.manual_seed(12)
    world, n = 4, 64 * 4 * 129
    shard = n // world
    planes = P2PPlane.fake(n * 2 + 4096, world, DEV)
    weights = [pl.alloc(n, torch.bfloat16) for pl in planes]
    kw = dict(kind=kind, lr=3e-3, alpha=8 / 11, step=3, kappa=0.85, clipsnr=2.0, eps=1e-8, gamma3=1.0, wd_factor=0.999,
              grad_scale=0.25, betas=(0.9, 0.95))
    clip = torch.tensor([0.8, 0.0], device=DEV)
    expect = torch.empty(n, device=DEV)
    for r, pl in enumerate(planes):
        p, g = torch.randn(shard, device=DEV), torch.randn(shard, device=DEV) * 1e-2
        m, v, tau = torch.randn(shard, device=DEV) * 1e-3, torch.rand(shard, device=DEV) * 1e-4, torch.rand(shard, device=DEV) * 0.6
        ref = [t.clone() for t in (p, g, m, v, tau)]
        pl.opt_step_push(p, g, m, v, tau, weights[r], r * shard, optim.make_hyper(**kw), clip)
        optim.fused_step(ref[0], ref[1], ref[2], ref[3], ref[4], None, clip_coef_t=clip, **kw)
        assert rel_err(p, ref[0]) < 1e-6 and rel_err(m, ref[2]) < 1e-6 and rel_err(v, ref[3]) < 1e-6
        expect[r * shard:(r + 1) * shard] = ref[0]
    for w in weights:        # every rank's resident copy now holds every shard
        assert rel_err(w, expect) < 8e-3


def test_p2p_push_f32_and_barrier_timeout():
    from adana_b200.parallel.p2p import P2PPlane

    planes = P2PPlane.fake(1 << 16, 2, DEV)
    dst = [pl.alloc(256, torch.float32) for pl in planes]
    src = torch.randn(64, device=DEV)
    planes[0].push_f32(src, dst[0], 128)
    for d in dst:
        assert torch.equal(d[128:192], src) and d[:128].abs().sum().item() == 0
    # a barrier whose peer never arrives gives up after its time limit and reports it through the status word
    planes[0].timeout_ns = int(0.2e9)
    planes[0].barrier()
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="peer flag"):
        _lib.check_status()


@pytest.mark.parametrize("wire", [torch.bfloat16, torch.float32], ids=["bf16_wire", "fp32_wire"])
def test_p2p_flagged_reduce_scatter_and_all_reduce_fake_peers(wire):
    """Per-unit ready flags instead of a barrier, bf16 or fp32 on the wire, fp32 sums.  All "ranks" are arenas on this
    GPU: every rank signals first (plain launches in stream order), so the waits inside the pulling kernels find their
    flags set; then a wait for a flag that nothing sets must give up within its limit, leave the output alone and report
    through the status word."""
    from adana_b200.parallel.p2p import P2PPlane

    torch.manual_seed(13)
    world, n = 4, 64 * 4 * 131
    shard = n // world
    planes = P2PPlane.fake(n * 8 + 8192, world, DEV)
    grads = [pl.alloc(n, torch.float32) for pl in planes]
    wires = [pl.alloc(n, torch.bfloat16) for pl in planes] if wire == torch.bfloat16 else grads
    for g, w in zip(grads, wires):
        g.copy_(torch.randn(n, device=DEV))
        if w is not g:
            optim.cast_f32_to_bf16(g, w)
    total = torch.stack([w.float() for w in wires]).sum(0)      # what the wire carries, summed in fp32
    unit, seq = 5, 7
    for pl in planes:
        pl.signal_unit(unit, seq)
    for r, pl in enumerate(planes):
        out = torch.zeros(shard, device=DEV)
        ss = torch.zeros(1, device=DEV)
        pl.reduce_scatter_unit(wires[r], r * shard, out, ss, unit, seq)
        assert rel_err(out, total[r * shard:(r + 1) * shard]) < 1e-6
        assert abs(ss.item() - out.double().pow(2).sum().item()) / ss.item() < 1e-4
    # all-reduce: rank r sums slice r and stores it into every rank's fp32 buffer (in place for an fp32 wire)
    for r, pl in enumerate(planes):
        pl.all_reduce_unit(wires[r], grads[r], r * shard, shard, unit, seq)
    for g in grads:
        assert rel_err(g, total) < 1e-6
    torch.cuda.synchronize()
    _lib.check_status()
    # a sequence number nobody has signalled: bounded wait, status word, output untouched
    planes[0].timeout_ns = int(0.2e9)
    out = torch.full((shard,), 3.0, device=DEV)
    planes[0].reduce_scatter_unit(wires[0], 0, out, None, unit, seq + 1)
    torch.cuda.synchronize()
    assert torch.equal(out, torch.full_like(out, 3.0))
    with pytest.raises(RuntimeError, match="peer flag"):
        _lib.check_status()


def test_newton_schulz_tcgen05_chain_matches_pytorch():
    from adana_b200.ops import muon_ns
    from adana_b200.optim.muon import newton_schulz5

    torch.manual_seed(5)
    for shape in ((256, 512), (768, 256), (384, 384)):
        G = torch.randn(*shape, device=DEV, dtype=torch.bfloat16)
        assert muon_ns.supported(G)
        before = _lib.launch_count()
        got = muon_ns.newton_schulz5_cuda(G, 5)
        assert _lib.launch_count() - before == 15                 # three GEMM launches per iteration, nothing else
        want = newton_schulz5(G.float(), 5)                       # fp32 oracle of the same iteration
        assert got.shape == G.shape
        err = (got.float() - want).norm() / want.norm()
        assert err < 0.05, (shape, float(err))
        sv = torch.linalg.svdvals(got.float())
        assert 0.5 < float(sv.median()) < 1.3


@pytest.mark.parametrize("hd,Hq,Hk,S", [(64, 4, 4, 256), (64, 4, 2, 512), (128, 2, 2, 256), (128, 4, 1, 384)])
def test_attention_jvp_matches_torch_func_jvp(hd, Hq, Hk, S):
    from adana_b200.ops import attention_native as an

    torch.manual_seed(17)
    B = 2
    T = B * S
    q, k, v = rnd(T, Hq, hd, scale=1.0), rnd(T, Hk, hd, scale=1.0), rnd(T, Hk, hd, scale=1.0)
    tq, tk, tv = rnd(T, Hq, hd, scale=1.0), rnd(T, Hk, hd, scale=1.0), rnd(T, Hk, hd, scale=1.0)
    out, tout = an.jvp(q, k, v, tq, tk, tv, B, S)
    ref_out, ref_tout = an.jvp_ref(q, k, v, tq, tk, tv, B, S)
    assert rel_err(out, ref_out) < 1.5e-2
    assert rel_err(tout, ref_tout) < 2.5e-2
    # the primal half agrees with the forward kernel
    fwd_out, _ = an.fwd(q, k, v, 0, hd, B, S, hd ** -0.5)
    assert rel_err(out, fwd_out) < 1e-2


@pytest.mark.parametrize("world,spr,d", [(2, 1, 64), (4, 2, 520), (8, 4, 2048)])
def test_p2p_all_to_all_pull_over_fake_peers(world, spr, d):
    """Variable-size all-to-all of rows (expert-parallel dispatch / combine) with every "rank" an arena on this GPU:
    all ranks publish, then each collects; checked against the permutation built with torch, and the reverse
    exchange must return every row to where it came from."""
    from adana_b200.parallel.p2p import P2PAllToAll, P2PPlane

    torch.manual_seed(41)
    n_seg = world * spr
    max_rows = 900
    planes = P2PPlane.fake(P2PAllToAll.arena_bytes(max_rows, d, torch.bfloat16, world, spr), world, DEV)
    a2a = [P2PAllToAll(pl, max_rows, d, torch.bfloat16, spr) for pl in planes]
    counts = [torch.randint(0, 40, (n_seg,), device=DEV) for _ in range(world)]
    counts[0][:spr] = 0                                   # an empty group
    rows = [rnd(int(c.sum()), d, scale=1.0) for c in counts]
    for r in range(world):
        a2a[r].publish(rows[r], counts[r])
    got = [a2a[r].collect() for r in range(world)]
    for me in range(world):
        parts, cexp = [], []
        for p in range(world):
            c = counts[p].view(world, spr)
            start = int(c[:me].sum())
            parts.append(rows[p][start:start + int(c[me].sum())])
            cexp.append(c[me])
        assert torch.equal(got[me][0], torch.cat(parts))
        assert torch.equal(got[me][1].long(), torch.cat(cexp))
    # reverse: publish what was received (table = received counts); everything returns in the original order
    for r in range(world):
        a2a[r].publish(got[r][0], got[r][1])
    for r in range(world):
        back, cback = a2a[r].collect(expect_rows=rows[r].shape[0])
        assert torch.equal(back, rows[r])
        assert torch.equal(cback.long(), counts[r])
    _lib.check_status()


@pytest.mark.parametrize("world,M,N,Kl", [(4, 1024, 512, 256), (4, 384, 384, 192), (8, 8192, 2304, 288), (2, 4096, 2304, 1152)])
def test_gemm_fused_with_reduce_scatter_over_fake_peers(world, M, N, Kl, gemm_mode):
    """Row-parallel linear whose epilogue does the reduce-scatter: every "rank" (here: one launch per rank on this
    GPU, the ranks' output buffers separate allocations) adds its partial product's rows into the buffer of the
    rank that owns them.  After all launches buffer r holds rows [r * M/world, ...) of the full product."""
    torch.manual_seed(31)
    K = world * Kl
    x, w = rnd(M, K), rnd(N, K)
    rows = M // world
    outs = [torch.zeros(rows, N, device=DEV) for _ in range(world)]
    for r in range(world):
        xr, wr = x[:, r * Kl:(r + 1) * Kl].contiguous(), w[:, r * Kl:(r + 1) * Kl].contiguous()
        gemm.linear_fwd_reduce_scatter(xr, wr, outs, rows, r, push=False)
    ref = x.float() @ w.float().t()
    got = torch.cat(outs, 0)
    assert rel_err(got, ref) < 5e-3
    # alpha and a pre-loaded residual: the epilogue adds, it never overwrites
    base = [torch.randn(rows, N, device=DEV) for _ in range(world)]
    outs2 = [b.clone() for b in base]
    for r in range(world):
        xr, wr = x[:, r * Kl:(r + 1) * Kl].contiguous(), w[:, r * Kl:(r + 1) * Kl].contiguous()
        gemm.linear_fwd_reduce_scatter(xr, wr, outs2, rows, r, alpha=0.5, push=False)
    assert rel_err(torch.cat(outs2, 0), torch.cat(base, 0) + 0.5 * ref) < 5e-3
    # push mode: bf16 partial rows stored into per-source slots at the owner, then summed in slot order
    slots = [torch.full((world, rows, N), float("nan"), device=DEV, dtype=torch.bfloat16) for _ in range(world)]
    for r in range(world):
        xr, wr = x[:, r * Kl:(r + 1) * Kl].contiguous(), w[:, r * Kl:(r + 1) * Kl].contiguous()
        gemm.linear_fwd_reduce_scatter(xr, wr, slots, rows, r, push=True)
    got = torch.cat([gemm.sum_slots(sl) for sl in slots], 0)
    assert rel_err(got, ref) < 6e-3
    part = torch.stack([(x[:, r * Kl:(r + 1) * Kl].float() @ w[:, r * Kl:(r + 1) * Kl].float().t()) for r in range(world)])
    assert rel_err(slots[0], part[:, :rows]) < 6e-3          # slot s of rank 0 = rank s's partial of rank 0's rows
    # pull-style reduce-scatter over whole bf16 partial matrices (one per "rank")
    partials = [part[r].bfloat16() for r in range(world)]
    for me in (0, world - 1):
        out = torch.empty(rows, N, device=DEV)
        gemm.reduce_scatter_partials(partials, me * rows, rows, N, N, out)
        assert rel_err(out, ref[me * rows:(me + 1) * rows]) < 6e-3
    lowp = torch.empty(rows, N, device=DEV, dtype=torch.bfloat16)
    withres = gemm.sum_slots(slots[1], resid=base[1], out_lowp=lowp)
    assert rel_err(withres, base[1] + ref[rows:2 * rows]) < 6e-3 and rel_err(lowp, withres) < 5e-3
    _lib.check_status()


@pytest.mark.parametrize("world,me,N,K", [(2, 0, 768, 512), (2, 1, 768, 512), (8, 3, 2304, 640), (8, 7, 6912, 512),
                                          (4, 2, 1280, 1152), (3, 1, 896, 576)])
def test_staged_gather_gemm_copies_each_remote_slice_once(world, me, N, K):
    """The staged variant: copier warps of the same kernel bring the slices other than `me` into a staging matrix,
    the tile order starts on slice `me`, and tiles on the other slices wait for their chunk's counter.  Shards are
    separate allocations on this GPU; the result has the bits of the plain CTA-pair kernel on the whole weight."""
    torch.manual_seed(23)
    M = 2048
    x, w = rnd(M, K), rnd(N, K)
    starts = gemm.tile_aligned_row_starts(N, world)
    cut = [w[a:b].clone() for a, b in zip(starts, starts[1:])]
    old = gemm.set_mode(3)
    try:
        ref_y = gemm.linear_fwd(x, w)
    finally:
        gemm.set_mode(old)
    for _ in range(3):   # the flag words are reused from launch to launch
        y = gemm.linear_fwd_gathered(x, cut, row_starts=starts, me=me, staged=True)
        assert torch.equal(y, ref_y)
    z, h = gemm.linear_gelu_fwd_gathered(x, cut, row_starts=starts, me=me, staged=True)
    assert torch.equal(z, ref_y) and rel_err(h, torch.nn.functional.gelu(x.float() @ w.float().t())) < 8e-3
    # dgrad: the contraction index is the sharded one and the k-loop starts on slice `me`
    dy = rnd(M, N)
    dx = gemm.linear_dgrad_gathered(dy, cut, None, K, row_starts=starts, me=me, staged=True)
    assert rel_err(dx, dy.float() @ w.float()) < 8e-3
    direct = gemm.linear_dgrad_gathered(dy, cut, None, K, row_starts=starts)
    assert rel_err(dx, direct) < 4e-3      # same products, summed in a rotated order
    # the dispatch on ShardedWeight takes the staged path by itself for tall inputs
    sw = gemm.ShardedWeight(cut, starts, N, K, local=cut, me=me)
    assert torch.equal(gemm.linear_fwd(x, sw), ref_y)
    _lib.check_status()


@pytest.mark.parametrize("world,rps", [(2, 96), (8, 96), (4, 352), (8, 864)])
def test_gather_gemm_reads_row_sharded_weights_in_place(world, rps):
    """The all-gather fused into the GEMM, with every rank's shard a separate allocation on this GPU.
    rps = rows per shard: a multiple of 32 but not of the 128-row half tile, so tiles straddle shards
    (32-row boxes) and, for the larger shards, also lie inside one (whole-tile boxes)."""
    torch.manual_seed(21)
    M, K = 1024, 512
    N = world * rps
    x, w = rnd(M, K), rnd(N, K)
    shards = [w[r * rps:(r + 1) * rps].clone() for r in range(world)]      # separate allocations
    ref = x.float() @ w.float().t()
    y = gemm.linear_fwd_gathered(x, shards, rps)
    assert y.shape == (M, N) and rel_err(y, ref) < 8e-3
    z, h = gemm.linear_gelu_fwd_gathered(x, shards, rps)
    assert rel_err(z, ref) < 8e-3 and rel_err(h, torch.nn.functional.gelu(ref)) < 8e-3
    # dgrad: the contraction index (rows of W) is the sharded one
    dy = rnd(M, N)
    dx = gemm.linear_dgrad_gathered(dy, shards, rps, K)
    assert rel_err(dx, dy.float() @ w.float()) < 8e-3
    # same bits as the plain CTA-pair kernel on the gathered weight
    old = gemm.set_mode(3)
    try:
        assert torch.equal(y, gemm.linear_fwd(x, w))
    finally:
        gemm.set_mode(old)
    # uneven slices cut on whole tiles: every B tile comes from one rank
    starts = gemm.tile_aligned_row_starts(N, world)
    assert starts[0] == 0 and starts[-1] == N and all(s % 128 == 0 for s in starts[:-1])
    if all(b > a for a, b in zip(starts, starts[1:])):
        cut = [w[a:b].clone() for a, b in zip(starts, starts[1:])]
        assert torch.equal(gemm.linear_fwd_gathered(x, cut, row_starts=starts), y)
        assert rel_err(gemm.linear_dgrad_gathered(dy, cut, None, K, row_starts=starts), dy.float() @ w.float()) < 8e-3


def test_muon_chain_kernels_with_fake_peers():
    """The four kernels around the Newton-Schulz GEMMs of distributed Muon, with four "ranks" that are buffers on one
    GPU (no flag waits: the launches run one after the other): momentum + staging + partial norms, pull + normalise,
    push to the holders, apply + weight push; against plain PyTorch in fp32."""
    import ctypes

    import numpy as np

    from adana_b200.parallel.dist_muon import SEG_DTYPE, _u64

    lib = _lib.lib()
    torch.manual_seed(11)
    world, parts_n = 4, int(lib.adana_muon_parts())
    slots = [("m0", (64, 96), 0, True), ("m1", (128, 64), 6144, True), ("vec", (100,), 14336, False)]
    padded = 14592
    shard = padded // world
    g = torch.randn(padded, device=DEV) * 0.1
    buf = torch.randn(padded, device=DEV) * 0.1
    p = torch.randn(padded, device=DEV)
    m1, m2 = torch.rand(padded, device=DEV) * 0.1, torch.rand(padded, device=DEV) * 0.01
    clip = torch.tensor([0.7, 0.0], device=DEV)
    gscale, mu, lr, wd, rms = 0.25, 0.9, (1e-2, 2e-2), (0.1, 0.0), 0.2
    b1, b2, eps, bias = 0.8, 0.99, 1e-8, 0.5
    stat = _lib.status_buffer(DEV).data_ptr()
    st = _lib.stream_ptr()
    # per-rank state
    ns = [torch.zeros(padded, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    upd = [torch.zeros(padded, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    wts = [torch.zeros(padded, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    parts = [torch.full((2 * parts_n,), 7.0, device=DEV) for _ in range(world)]
    gs, bs, ps, m1s, m2s, tables = [], [], [], [], [], []
    for r in range(world):
        lo, hi = r * shard, (r + 1) * shard
        rows = []
        for i, (_, shape, off, decay) in enumerate(slots):
            n = int(np.prod(shape))
            a, b = max(off, lo), min(off + n, hi)
            if len(shape) == 2:
                a, b = (a - lo, b - lo) if a < b else (0, 0)
                rows.append((a, b, 0, 0 if decay else 1, rms * max(shape) ** 0.5, i))
            elif a < b:
                rows.append((a - lo, b - lo, 1, 0 if decay else 1, 0.0, 0))
        t = torch.from_numpy(np.array(rows, dtype=SEG_DTYPE).view(np.uint8).copy()).to(DEV)
        tables.append((t, len(rows), max(x[1] - x[0] for x in rows)))
        gs.append(g[lo:hi].clone()); bs.append(buf[lo:hi].clone()); ps.append(p[lo:hi].clone())
        m1s.append(m1[lo:hi].clone()); m2s.append(m2[lo:hi].clone())
        _lib.check_rc(lib.adana_muon_momentum(gs[r].data_ptr(), bs[r].data_ptr(), ns[r].data_ptr() + 2 * lo, t.data_ptr(), 2,
                                              clip.data_ptr(), gscale, mu, 1, parts[r].data_ptr(), st), "momentum")
    geff = g * gscale * 0.7
    buf_ref = mu * buf + geff
    ns_ref = (geff + mu * buf_ref).bfloat16()
    for i, (_, shape, off, _) in enumerate(slots[:2]):
        n = shape[0] * shape[1]
        assert_close(torch.cat(bs)[off:off + n], buf_ref[off:off + n], 1e-5, 1e-6, "momentum buffer")
        X = torch.empty(n, dtype=torch.bfloat16, device=DEV)
        _lib.check_rc(lib.adana_muon_pull(_u64([t.data_ptr() for t in ns]), _u64([t.data_ptr() for t in parts]), world, shard,
                                          off, n, i, 1e-7, X.data_ptr(), 0, 0, 0, stat, st), "pull")
        want = ns_ref[off:off + n].float()
        want = want / (want.norm() + 1e-7)
        assert_close(X.float(), want, 1e-2, 1e-5, "pulled and normalised matrix")
        _lib.check_rc(lib.adana_muon_push(X.data_ptr(), _u64([t.data_ptr() for t in upd]), world, shard, off, n, st), "push")
    hyper = (ctypes.c_float * 9)(lr[0], lr[1], wd[0], wd[1], b1, b2, eps, bias, gscale)
    for r in range(world):
        lo = r * shard
        t, n_segs, longest = tables[r]
        _lib.check_rc(lib.adana_muon_apply(ps[r].data_ptr(), gs[r].data_ptr(), upd[r].data_ptr() + 2 * lo, m1s[r].data_ptr(),
                                           m2s[r].data_ptr(), t.data_ptr(), n_segs, hyper, clip.data_ptr(),
                                           _u64([w.data_ptr() for w in wts]), world, lo, longest, 0, 0, world, 0, stat, st), "apply")
    torch.cuda.synchronize()
    _lib.check_status()
    got = torch.cat(ps)
    want_p = p.clone()
    for i, (_, shape, off, _) in enumerate(slots[:2]):
        n = shape[0] * shape[1]
        x = ns_ref[off:off + n].float()
        x = (x / (x.norm() + 1e-7)).bfloat16().float()
        want_p[off:off + n] = p[off:off + n] * (1 - lr[0] * wd[0]) - lr[0] * rms * max(shape) ** 0.5 * x
    off, n = slots[2][2], 100
    ge = geff[off:off + n]
    a = m1[off:off + n] + (1 - b1) * (ge - m1[off:off + n])
    b = m2[off:off + n] + (1 - b2) * (ge * ge - m2[off:off + n])
    want_p[off:off + n] = p[off:off + n] * (1 - lr[1] * wd[1]) - lr[1] / bias * a / (eps + b.sqrt())
    used = torch.zeros(padded, dtype=torch.bool, device=DEV)
    for _, shape, off, _ in slots:
        used[off:off + int(np.prod(shape))] = True
    assert_close(got[used], want_p[used], 1e-2, 1e-4, "updated parameters")
    assert torch.equal(got[~used], p[~used])                                   # padding is never touched
    assert_close(torch.cat(m1s)[off:off + n], a, 1e-5, 1e-7, "AdamW first moment")
    for w in wts:                                                              # every rank received every new weight
        assert torch.equal(w[used], got[used].bfloat16())
