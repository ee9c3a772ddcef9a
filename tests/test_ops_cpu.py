"""Host-side logic of the op wrappers that needs no GPU: reference paths and argument policies."""
import pytest
import torch

from adana_b200.ops import gemm


def test_sum_slots_reference_path_adds_in_fp32_with_residual():
    torch.manual_seed(0)
    slots = torch.randn(4, 6, 16).bfloat16()
    resid = torch.randn(6, 16)
    lowp = torch.empty(6, 16, dtype=torch.bfloat16)
    out = gemm.sum_slots(slots, resid=resid, out_lowp=lowp)
    assert out.dtype == torch.float32
    assert torch.allclose(out, slots.float().sum(0) + resid, atol=1e-6)
    assert torch.allclose(lowp.float(), out, atol=2e-2, rtol=1e-2)


def test_tile_aligned_row_starts_cover_the_rows_on_whole_tiles():
    for rows, world in ((6912, 8), (2304, 8), (9216, 2), (1280, 4), (896, 3), (128, 1)):
        s = gemm.tile_aligned_row_starts(rows, world)
        assert len(s) == world + 1 and s[0] == 0 and s[-1] == rows
        assert all(b >= a for a, b in zip(s, s[1:])) and all(v % 128 == 0 for v in s[:-1])
        sizes = [b - a for a, b in zip(s, s[1:])]
        assert max(sizes) - min(sizes) <= 128 + (128 - rows % 128) % 128      # balanced to within one tile


def test_sharded_weight_cpu_path_uses_the_full_matrix():
    torch.manual_seed(1)
    w = torch.randn(256, 32).bfloat16()
    starts = gemm.tile_aligned_row_starts(256, 2)
    views = [w[a:b] for a, b in zip(starts, starts[1:])]
    sw = gemm.ShardedWeight(views, starts, 256, 32, local=views, me=1)
    x = torch.randn(8, 32).bfloat16()
    assert torch.equal(gemm.linear_fwd(x, sw), gemm.linear_fwd(x, w))
    assert sw.me == 1 and torch.equal(sw.full(), w)
    with pytest.raises(RuntimeError):
        gemm.ShardedWeight([0, 0], starts, 256, 32).full()
