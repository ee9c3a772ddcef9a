"""The allocation-free norm backward (`adana_norm_bwd_static_scratch`), called through the exported C symbol.

Collected last (file name) so that it also runs after every other GPU test has used the library; it passes on
its own as well.  The existing entry point (`adana_norm_bwd` + `adana_colsum_f32` through `ops.norm.norm_bwd`)
is the reference: both run the same kernels with the same grid, so results agree to rounding.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_COLS = 4096
E_COLS = -21


def _symbol():
    from adana_b200.ops import _lib

    cdll = ctypes.CDLL(str(_lib.lib_path()))           # the plain shared object, not the Python-side proxy
    fn = cdll.adana_norm_bwd_static_scratch
    vp, i = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [vp, i, vp, i, vp, vp, vp, vp, i, vp, i, i, i, i, vp, vp]
    fn.restype = i
    return fn


def _case(rows, cols, kind, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, cols, device="cuda", generator=g)
    dy = (torch.randn(rows, cols, device="cuda", generator=g) * 0.3).to(torch.bfloat16)
    w = 1.0 + 0.1 * torch.randn(cols, device="cuda", generator=g)
    if kind == 0:
        mean = x.mean(-1)
        rstd = (x.var(-1, unbiased=False) + 1e-5).rsqrt()
    else:
        mean = torch.zeros(rows, device="cuda")
        rstd = (x.square().mean(-1) + 1e-5).rsqrt()
    return x, dy, w, mean.contiguous(), rstd.contiguous()


@pytest.mark.parametrize("kind", [0, 1])
def test_static_scratch_matches_existing_entry_point_twice_in_a_row(kind):
    from adana_b200.ops import norm

    fn = _symbol()
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back on one stream: the second must not see the first one's partial rows
    for seed, (rows, cols) in enumerate([(3000, 2304), (777, 1024)]):
        x, dy, w, mean, rstd = _case(rows, cols, kind, seed)
        dx = torch.empty(rows, cols, device="cuda")
        dw = torch.empty(cols, device="cuda")
        rc = fn(dy.data_ptr(), 1, x.data_ptr(), 0, w.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(), 0,
                dw.data_ptr(), 0, rows, cols, kind, None, stream)
        assert rc == 0
        want_dx, want_dw = norm.norm_bwd(dy, x, w, mean, rstd, kind=kind)
        torch.cuda.synchronize()
        assert torch.allclose(dx, want_dx, rtol=1e-6, atol=1e-7)
        # (the two entry points cut the rows into different numbers of partial sums: equal up to fp32 summation order)
        assert torch.allclose(dw, want_dw, rtol=1e-5, atol=1e-4)
        ref_dx, ref_dw = norm.norm_bwd_ref(dy, x, w, mean, rstd, kind)      # plain PyTorch fp32 of the same op
        assert torch.allclose(dx, ref_dx, rtol=1e-3, atol=1e-4)
        assert torch.allclose(dw, ref_dw, rtol=1e-3, atol=2e-2)


def test_static_scratch_accumulates_and_rejects_oversize():
    from adana_b200.ops import norm

    fn = _symbol()
    stream = torch.cuda.current_stream().cuda_stream
    rows, cols = 512, 768
    x, dy, w, mean, rstd = _case(rows, cols, 0, 9)
    dx = torch.ones(rows, cols, device="cuda")
    dw = torch.full((cols,), 2.0, device="cuda")
    assert fn(dy.data_ptr(), 1, x.data_ptr(), 0, w.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(), 1,
              dw.data_ptr(), 1, rows, cols, 0, None, stream) == 0
    want_dx, want_dw = norm.norm_bwd(dy, x, w, mean, rstd, kind=0)
    torch.cuda.synchronize()
    assert torch.allclose(dx, want_dx + 1.0, rtol=1e-5, atol=1e-6)
    assert torch.allclose(dw, want_dw + 2.0, rtol=1e-5, atol=1e-4)
    # beyond the built-in scratch: refused before any launch, outputs untouched
    before = dw.clone()
    big = MAX_COLS + 4
    assert fn(dy.data_ptr(), 1, x.data_ptr(), 0, w.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(), 0,
              dw.data_ptr(), 0, 4, big, 0, None, stream) == E_COLS
    assert fn(dy.data_ptr(), 1, x.data_ptr(), 0, w.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(), 0,
              dw.data_ptr(), 0, 4, 770, 0, None, stream) == E_COLS
    torch.cuda.synchronize()
    assert torch.equal(dw, before)


def test_static_scratch_rmsnorm_without_mean_and_empty_batch():
    """RMSNorm never reads `mean`, so a caller may pass NULL; zero rows leave dw = 0 (or untouched when accumulating)."""
    from adana_b200.ops import norm

    fn = _symbol()
    stream = torch.cuda.current_stream().cuda_stream
    rows, cols = 640, 512
    x, dy, w, mean, rstd = _case(rows, cols, 1, 3)
    dx = torch.empty(rows, cols, device="cuda")
    dw = torch.empty(cols, device="cuda")
    assert fn(dy.data_ptr(), 1, x.data_ptr(), 0, w.data_ptr(), None, rstd.data_ptr(), dx.data_ptr(), 0,
              dw.data_ptr(), 0, rows, cols, 1, None, stream) == 0
    want_dx, want_dw = norm.norm_bwd(dy, x, w, mean, rstd, kind=1)
    torch.cuda.synchronize()
    assert torch.allclose(dx, want_dx, rtol=1e-6, atol=1e-7)
    assert torch.allclose(dw, want_dw, rtol=1e-5, atol=1e-4)
    # LayerNorm does read it: NULL is refused
    assert fn(dy.data_ptr(), 1, x.data_ptr(), 0, w.data_ptr(), None, rstd.data_ptr(), dx.data_ptr(), 0,
              dw.data_ptr(), 0, rows, cols, 0, None, stream) == -22
    dw.fill_(5.0)
    assert fn(dy.data_ptr(), 1, x.data_ptr(), 0, w.data_ptr(), None, rstd.data_ptr(), dx.data_ptr(), 0,
              dw.data_ptr(), 1, 0, cols, 1, None, stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(dw, torch.full_like(dw, 5.0))
    assert fn(dy.data_ptr(), 1, x.data_ptr(), 0, w.data_ptr(), None, rstd.data_ptr(), dx.data_ptr(), 0,
              dw.data_ptr(), 0, 0, cols, 1, None, stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(dw, torch.zeros_like(dw))
