"""Malformed shapes are a host matter: the C entry points refuse them with a negative return code BEFORE any launch
(nothing is enqueued, no pointer is touched), so these cases run without a GPU.  No test hands a device an argument
it is expected to reject there."""
import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
from hypothesis import given, settings
from hypothesis import strategies as st

from adana_b200.ops import _lib


@pytest.fixture(scope="module")
def cdll():
    path = _lib.lib_path()
    if not path.exists():
        from adana_b200 import build

        build.build()
    lib = ctypes.CDLL(str(path))
    P, I, L, F = c_void_p, c_int, c_longlong, c_float
    lib.adana_attn_fwd.argtypes = [P, P, P, L, I, P, P, I, I, I, I, I, F, P, P]
    lib.adana_attn_bwd.argtypes = [P, P, P, L, I, P, P, P, P, P, P, L, I, P, I, I, I, I, I, F, P, P]
    lib.adana_attn_jvp.argtypes = [P, P, P, P, P, P, P, P, I, I, I, I, I, F, P, P]
    lib.adana_p2p_reduce_scatter_flag.argtypes = [P, I, P, ctypes.c_uint, I, L, L, P, P, ctypes.c_ulonglong, P, P]
    lib.adana_p2p_all_reduce_flag.argtypes = [P, I, P, P, ctypes.c_uint, I, L, L, P, ctypes.c_ulonglong, P, P]
    lib.adana_p2p_opt_step_push.argtypes = [P, P, P, P, P, P, I, L, L, P, P, P]
    lib.adana_ce_fwd_bwd.argtypes = [P, L, P, I, I, F, F, P, L, P, P, P]
    lib.adana_ce_fwd_bwd_bf16.argtypes = [P, L, P, I, I, F, F, P, L, P, P, P]
    lib.adana_norm_bwd_static_scratch.argtypes = [P, I, P, I, P, P, P, P, I, P, I, I, I, I, P, P]
    for name in ("adana_attn_fwd", "adana_attn_bwd", "adana_attn_jvp", "adana_p2p_reduce_scatter_flag",
                 "adana_p2p_all_reduce_flag", "adana_p2p_opt_step_push", "adana_ce_fwd_bwd", "adana_ce_fwd_bwd_bf16",
                 "adana_norm_bwd_static_scratch"):
        getattr(lib, name).restype = c_int
    return lib


_bad_attention = st.one_of(
    st.tuples(st.integers(1, 4), st.integers(1, 64).map(lambda k: k * 128), st.integers(1, 8), st.just(1),
              st.integers(1, 512).filter(lambda h: h not in (64, 128))),                 # head_dim other than 64 / 128
    st.tuples(st.integers(1, 4), st.integers(1, 8192).filter(lambda s: s % 128), st.integers(1, 8), st.just(1),
              st.sampled_from([64, 128])),                                                # S not a multiple of the tile
    st.tuples(st.integers(1, 4), st.integers(1, 64).map(lambda k: k * 128), st.sampled_from([3, 5, 7, 9]), st.just(2),
              st.sampled_from([64, 128])),                                                # query heads not a multiple of KV heads
)


@settings(max_examples=60, deadline=None)
@given(_bad_attention)
def test_attention_entry_points_refuse_bad_shapes_before_any_launch(cdll, case):
    B, S, Hq, Hk, hd = case
    assert cdll.adana_attn_fwd(None, None, None, 0, 0, None, None, B, S, Hq, Hk, hd, 0.125, None, None) == -1
    assert cdll.adana_attn_bwd(None, None, None, 0, 0, None, None, None, None, None, None, 0, 0, None, B, S, Hq, Hk, hd,
                               0.125, None, None) == -1
    assert cdll.adana_attn_jvp(None, None, None, None, None, None, None, None, B, S, Hq, Hk, hd, 0.125, None, None) < 0


@settings(max_examples=60, deadline=None)
@given(st.integers(-3, 20), st.integers(0, 1 << 20), st.integers(0, 1 << 20))
def test_peer_collectives_refuse_bad_world_and_misaligned_ranges(cdll, world, off, n):
    bad = world < 1 or world > 8 or (n & 7) or (off & 7)
    if not bad:
        return                  # a valid range would be launched: out of scope here
    assert cdll.adana_p2p_reduce_scatter_flag(None, 1, None, 1, world, off, n, None, None, 10 ** 9, None, None) == -1
    assert cdll.adana_p2p_all_reduce_flag(None, 0, None, None, 1, world, off, n, None, 10 ** 9, None, None) == -1
    assert cdll.adana_p2p_opt_step_push(None, None, None, None, None, None, world, off, n, None, None, None) == -1


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 4096), st.integers(1, 100000))
def test_cross_entropy_and_static_norm_refuse_unaligned_widths(cdll, rows, vocab):
    if vocab % 4:
        assert cdll.adana_ce_fwd_bwd(None, vocab, None, rows, vocab, 0.0, 1.0, None, vocab, None, None, None) == -1
    if vocab % 8:
        assert cdll.adana_ce_fwd_bwd_bf16(None, vocab, None, rows, vocab, 0.0, 1.0, None, vocab, None, None, None) == -1
    if vocab % 4 or vocab > 4096:
        assert cdll.adana_norm_bwd_static_scratch(None, 1, None, 0, None, None, None, None, 0, None, 0, rows, vocab, 0,
                                                  None, None) == -21
