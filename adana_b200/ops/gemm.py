"""bf16 GEMMs on the tcgen05 tensor cores (csrc/gemm_tcgen05.cu) with fused epilogues.

`gemm()` is the thin wrapper over the C entry point; `linear_fwd / linear_dgrad /
linear_wgrad` name the three GEMMs of an `nn.Linear` so that callers never transpose a
tensor in memory: the kernel reads MN-major operands directly.

Each function has a PyTorch fp32-accumulate reference (`*_ref`) that runs on CPU and is
what the GPU tests compare against.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib

EPI_BF16, EPI_GELU_DUAL, EPI_RESID_F32, EPI_DGELU, EPI_F32, EPI_SWIGLU, EPI_DSWIGLU, EPI_AXPBY_BF16 = range(8)


MODE_AUTO, MODE_SINGLE_CTA, MODE_CTA_PAIR = 0, 1, 2


def set_mode(mode: int) -> int:
    """Tile policy of the GEMM kernel: MODE_AUTO picks per shape between one CTA per 128x256 tile and a CTA
    pair (cta_group::2) per 256x256 tile.  Returns the previous mode."""
    return _lib.lib().adana_gemm_set_mode(int(mode))


class ShardedWeight:
    """A weight matrix [N, K] (bf16) that is NOT held in one piece: rank r holds rows [row_starts[r], row_starts[r+1])
    at address `ptrs[r]` (its own memory or a peer's).  `linear_fwd`, `linear_gelu_fwd`, `linear_resid_fwd`,
    `linear_dgrad` and `linear_dgrad_dgelu` accept it in place of a tensor and run the gathering GEMM, which fetches
    every B tile from its owner.  `local` optionally keeps this process's tensors alive (and serves the CPU path).
    `me` names the slice that lives in this process's own memory: with it the GEMM brings the other slices over the
    link once into a staging matrix (inside the same kernel) instead of re-fetching them per row tile."""

    def __init__(self, ptrs, row_starts, N: int, K: int, local=None, me=None):
        import ctypes

        vals = [int(p.data_ptr()) if torch.is_tensor(p) else int(p) for p in ptrs]
        self.ptrs = (ctypes.c_uint64 * len(vals))(*vals)
        self.row_starts = [int(v) for v in row_starts]
        assert len(self.row_starts) == len(vals) + 1 and self.row_starts[0] == 0 and self.row_starts[-1] == N
        self.shape = (N, K)
        self.local = local
        self.me = me

    def full(self) -> torch.Tensor:
        """The gathered matrix, from the local tensors (single-process use and CPU reference path)."""
        if self.local is None or len(self.local) != len(self.row_starts) - 1:
            raise RuntimeError("this ShardedWeight has no local copy of every slice")
        return torch.cat([t.reshape(-1, self.shape[1]) for t in self.local], 0)


def _check2d(t: torch.Tensor, name: str):
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be 2-D with a contiguous last dimension, got {tuple(t.shape)} / {t.stride()}")
    if t.dtype != torch.bfloat16:
        raise ValueError(f"{name} must be bf16")
    if t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
        raise ValueError(f"{name}: row pitch must be a multiple of 8 elements and the base 16-byte aligned")


def gemm(A, B, C, *, M, N, K, a_mn=False, b_mn=False, epi=EPI_BF16, C2=None, R=None,
         alpha=1.0, beta=0.0, b_off2=0):
    """C = epilogue(A · Bᵀ) on the tensor cores; all tensors are pre-allocated by the caller."""
    _check2d(A, "A")
    _check2d(B, "B")
    lib = _lib.lib()
    rc = lib.adana_gemm_bf16(
        A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K,
        A.stride(0), B.stride(0), C.stride(0), int(a_mn), int(b_mn), int(epi),
        _lib.ptr(C2), 0 if C2 is None else C2.stride(0),
        _lib.ptr(R), 0 if R is None else R.stride(0),
        float(alpha), float(beta), int(b_off2),
        _lib.status_buffer(A.device).data_ptr(), _lib.stream_ptr())
    _lib.check_rc(rc, "adana_gemm_bf16")
    return C


# ----------------------------------------------------------------------------------------------
# nn.Linear GEMMs: x [M,K] (bf16), w [N,K] (bf16, the nn.Linear weight), dy [M,N] (bf16)
# ----------------------------------------------------------------------------------------------
def use_cuda(*ts) -> bool:
    """The tcgen05 path: CUDA tensors whose two GEMM operands (the first two arguments) are bf16; anything else (fp32
    compute on a GPU included) takes the PyTorch fp32 path of the same op."""
    return (all(t is None or t.is_cuda for t in ts) and _lib.available()
            and all(torch.is_tensor(t) and t.dtype == torch.bfloat16 for t in ts[:2]))


def linear_fwd(x, w, out=None):
    if isinstance(w, ShardedWeight):
        if not (x.is_cuda and _lib.available()):
            return linear_fwd(x, w.full(), out)
        return gather_gemm(x, w.ptrs, None, w.shape[0], ldb=w.shape[1], out=out, row_starts=w.row_starts, me=w.me)
    M, K = x.shape
    N = w.shape[0]
    if not use_cuda(x, w):
        r = (x.float() @ w.float().t()).to(x.dtype)
        if out is not None:
            out.copy_(r)
            return out
        return r
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    return gemm(x, w, out, M=M, N=N, K=K)


def linear_fwd_f32(x, w, out=None, alpha=1.0):
    """fp32 output (used for the logits chunks of the fused cross-entropy)."""
    M, K = x.shape
    N = w.shape[0]
    if not use_cuda(x, w):
        return (x.float() @ w.float().t()) * alpha
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    return gemm(x, w, out, M=M, N=N, K=K, epi=EPI_F32, alpha=alpha, beta=0.0)


def linear_gelu_fwd(x, w):
    """Returns (z, gelu(z)) in one pass: z is kept for backward, gelu(z) feeds the next GEMM."""
    if isinstance(w, ShardedWeight):
        if not (x.is_cuda and _lib.available()):
            return linear_gelu_fwd(x, w.full())
        z = torch.empty((x.shape[0], w.shape[0]), dtype=torch.bfloat16, device=x.device)
        h = torch.empty_like(z)
        gather_gemm(x, w.ptrs, None, w.shape[0], ldb=w.shape[1], epi=EPI_GELU_DUAL, out=z, C2=h, row_starts=w.row_starts, me=w.me)
        return z, h
    M, K = x.shape
    N = w.shape[0]
    if not use_cuda(x, w):
        z = (x.float() @ w.float().t())
        return z.to(x.dtype), F.gelu(z).to(x.dtype)
    z = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    h = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    gemm(x, w, z, M=M, N=N, K=K, epi=EPI_GELU_DUAL, C2=h)
    return z, h


def linear_resid_fwd(x, w, resid, alpha=1.0, out=None):
    """out(f32) = resid(f32) + alpha * x·wᵀ ; `out` may alias `resid`."""
    if isinstance(w, ShardedWeight):
        if not (x.is_cuda and _lib.available()):
            return linear_resid_fwd(x, w.full(), resid, alpha, out)
        if out is None:
            out = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float32, device=x.device)
        return gather_gemm(x, w.ptrs, None, w.shape[0], ldb=w.shape[1], epi=EPI_RESID_F32, out=out, R=resid, alpha=alpha,
                           row_starts=w.row_starts, me=w.me)
    M, K = x.shape
    N = w.shape[0]
    if not use_cuda(x, w, resid):
        r = resid + alpha * (x.float() @ w.float().t())
        if out is not None:
            out.copy_(r)
            return out
        return r
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    return gemm(x, w, out, M=M, N=N, K=K, epi=EPI_RESID_F32, R=resid, alpha=alpha)


def linear_swiglu_fwd(x, w_gu):
    """w_gu = [gate rows; up rows] ([2*H, K]).  Returns (gu [M,2H] pre-activations, h [M,H])."""
    M, K = x.shape
    H = w_gu.shape[0] // 2
    if not use_cuda(x, w_gu):
        gu = x.float() @ w_gu.float().t()
        g, u = gu[:, :H], gu[:, H:]
        return gu.to(x.dtype), (F.silu(g) * u).to(x.dtype)
    gu = torch.empty((M, 2 * H), dtype=torch.bfloat16, device=x.device)
    h = torch.empty((M, H), dtype=torch.bfloat16, device=x.device)
    gemm(x, w_gu, gu, M=M, N=H, K=K, epi=EPI_SWIGLU, C2=h, b_off2=H)
    return gu, h


def linear_dgrad(dy, w, out=None, alpha=1.0):
    """dx [M,K] = alpha * dy [M,N] · w [N,K]."""
    if isinstance(w, ShardedWeight):
        if not (dy.is_cuda and _lib.available()):
            return linear_dgrad(dy, w.full(), out, alpha)
        return gather_gemm(dy, w.ptrs, None, w.shape[1], ldb=w.shape[1], b_mn=True, out=out, alpha=alpha,
                           row_starts=w.row_starts, me=w.me)
    M, N = dy.shape
    K = w.shape[1]
    if not use_cuda(dy, w):
        r = (alpha * (dy.float() @ w.float())).to(dy.dtype)
        if out is not None:
            out.copy_(r)
            return out
        return r
    if out is None:
        out = torch.empty((M, K), dtype=torch.bfloat16, device=dy.device)
    return gemm(dy, w, out, M=M, N=K, K=N, b_mn=True, alpha=alpha)


def linear_dgrad_f32(dy, w, out=None, beta=0.0, resid=None):
    """fp32 dx; with `resid` computes resid + dy·w (gradient of a residual branch)."""
    M, N = dy.shape
    K = w.shape[1]
    if not use_cuda(dy, w):
        r = dy.float() @ w.float()
        if resid is not None:
            return resid + r
        return r if out is None or beta == 0.0 else beta * out + r
    if out is None:
        out = torch.empty((M, K), dtype=torch.float32, device=dy.device)
    if resid is not None:
        return gemm(dy, w, out, M=M, N=K, K=N, b_mn=True, epi=EPI_RESID_F32, R=resid)
    return gemm(dy, w, out, M=M, N=K, K=N, b_mn=True, epi=EPI_F32, beta=beta)


def linear_dgrad_dgelu(dy, w, z, alpha=1.0):
    """dz = alpha * (dy · w) * gelu'(z): gradient through `gelu` fused in the dgrad epilogue."""
    if isinstance(w, ShardedWeight):
        if not (dy.is_cuda and _lib.available()):
            return linear_dgrad_dgelu(dy, w.full(), z, alpha)
        out = torch.empty((dy.shape[0], w.shape[1]), dtype=torch.bfloat16, device=dy.device)
        return gather_gemm(dy, w.ptrs, None, w.shape[1], ldb=w.shape[1], b_mn=True, epi=EPI_DGELU, out=out, R=z, alpha=alpha,
                           row_starts=w.row_starts, me=w.me)
    M, N = dy.shape
    K = w.shape[1]
    if not use_cuda(dy, w, z):
        dh = dy.float() @ w.float()
        zf = z.float().requires_grad_(True)
        with torch.enable_grad():
            g, = torch.autograd.grad(F.gelu(zf).sum(), zf)
        return (alpha * dh * g).to(dy.dtype)
    out = torch.empty((M, K), dtype=torch.bfloat16, device=dy.device)
    return gemm(dy, w, out, M=M, N=K, K=N, b_mn=True, epi=EPI_DGELU, R=z, alpha=alpha)


def linear_dgrad_dswiglu(dy, w_down, gu, alpha=1.0):
    """d[gate|up] = swiglu'(gate, up) ∘ alpha (dy · w_down): w_down [d, H], gu [M, 2H]."""
    M, N = dy.shape
    H = w_down.shape[1]
    if not use_cuda(dy, w_down, gu):
        dh = alpha * (dy.float() @ w_down.float())
        g, u = gu[:, :H].float(), gu[:, H:].float()
        s = torch.sigmoid(g)
        dg = dh * u * s * (1 + g * (1 - s))
        du = dh * g * s
        return torch.cat([dg, du], dim=1).to(dy.dtype)
    out = torch.empty((M, 2 * H), dtype=torch.bfloat16, device=dy.device)
    return gemm(dy, w_down, out, M=M, N=H, K=N, b_mn=True, epi=EPI_DSWIGLU, R=gu, b_off2=H, alpha=alpha)


def linear_wgrad(dy, x, out=None, accumulate=False, alpha=1.0):
    """dw [N,K] (fp32) (+)= dyᵀ [N,M] · x [M,K]; both operands are read as stored."""
    M, N = dy.shape
    K = x.shape[1]
    if not use_cuda(dy, x):
        r = alpha * (dy.float().t() @ x.float())
        if out is None:
            return r
        if accumulate:
            out += r
        else:
            out.copy_(r)
        return out
    if out is None:
        out = torch.empty((N, K), dtype=torch.float32, device=dy.device)
        accumulate = False
    return gemm(dy, x, out, M=N, N=K, K=M, a_mn=True, b_mn=True, epi=EPI_F32,
                alpha=alpha, beta=1.0 if accumulate else 0.0)


# ----------------------------------------------------------------------------------------------
# All-gather fused into the GEMM: the weight is row-sharded over ranks.  Tall inputs use the staged kernel (copier
# warps of the GEMM bring each remote slice over the link once into a staging matrix while the tiles of the local
# slice run); short inputs fetch every B tile straight from its owner.  Also here: the row-parallel GEMM with the
# reduce-scatter of its partial products.
# ----------------------------------------------------------------------------------------------
def _ptr_array(shards):
    """list of tensors / ints, or a ready ctypes array -> (c_uint64 array, count)."""
    import ctypes

    if isinstance(shards, ctypes.Array):
        return shards, len(shards)
    vals = [int(s.data_ptr()) if torch.is_tensor(s) else int(s) for s in shards]
    return (ctypes.c_uint64 * len(vals))(*vals), len(vals)


def tile_aligned_row_starts(n_rows: int, world: int, tile: int = 128):
    """Split `n_rows` weight rows over `world` ranks on multiples of `tile` (the last slice takes the remainder), so
    that every B tile of the gathering GEMM lies inside one rank's slice.  Returns world + 1 offsets."""
    tiles = (n_rows + tile - 1) // tile
    base, extra = divmod(tiles, world)
    starts, pos = [0], 0
    for r in range(world):
        pos = min(n_rows, pos + (base + (1 if r < extra else 0)) * tile)
        starts.append(pos)
    return starts


_stage_ws = {}
STAGE_MIN_ROWS = 512     # below this the remote tiles are used by at most two row tiles: fetch them directly


def _stage_workspace(device, nbytes: int):
    """(staging bytes, flag words) of `device`, grown on demand and shared by every staged gather GEMM there: such
    launches must therefore be ordered on one stream, which the engine's compute stream does."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    ws = _stage_ws.get(key)
    if ws is None or ws[0].numel() < nbytes:
        ws = (torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device),
              torch.zeros(64 + 8 * 4096, dtype=torch.int32, device=device))
        _stage_ws[key] = ws
    return ws


def gather_gemm(x, shards, rows_per_shard, N, *, ldb, b_mn=False, epi=EPI_BF16, out=None, C2=None, R=None, alpha=1.0,
                out_dtype=torch.bfloat16, row_starts=None, me=None, staged=None):
    """C[M,N] = epi(x · Wᵀ) (b_mn False, W [N,K] row-sharded) or epi(x · W) (b_mn True, W [K,N] row-sharded).
    `row_starts` (world + 1 offsets, multiples of 32) gives uneven slices; otherwise every slice has
    `rows_per_shard` rows.  `me`: the slice in this process's own memory.  `staged` (default: whenever `me` is
    given, the slices are cut on whole tiles and x has at least STAGE_MIN_ROWS rows) copies the other slices once
    into a local staging matrix inside the kernel; otherwise every tile is fetched from its owner on each use."""
    import ctypes

    _check2d(x, "x")
    M, K = x.shape
    arr, n = _ptr_array(shards)
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    starts = None if row_starts is None else (ctypes.c_int * (n + 1))(*[int(v) for v in row_starts])
    w_rows = K if b_mn else N
    cut = 64 if b_mn else 128
    bounds = list(row_starts) if row_starts is not None else [r * rows_per_shard for r in range(n + 1)]
    can_stage = me is not None and all(v % cut == 0 for v in bounds[:-1]) and bounds[-1] == w_rows and w_rows // cut < 4000
    if staged is None:
        staged = can_stage and M >= STAGE_MIN_ROWS and n > 1
    elif staged and not can_stage:
        raise ValueError("staged gather needs `me` and slices cut on multiples of %d rows" % cut)
    stage_ptr = flags_ptr = None
    if staged:
        stage, flags = _stage_workspace(x.device, w_rows * int(ldb) * 2)
        stage_ptr, flags_ptr = stage.data_ptr(), flags.data_ptr()
    rc = _lib.lib().adana_gemm_bf16_gather(
        x.data_ptr(), arr, n, int(rows_per_shard or 0), starts, out.data_ptr(), M, N, K, x.stride(0), int(ldb),
        out.stride(0), int(b_mn), int(epi), _lib.ptr(C2), 0 if C2 is None else C2.stride(0), _lib.ptr(R),
        0 if R is None else R.stride(0), float(alpha), int(me or 0), stage_ptr, flags_ptr,
        _lib.status_buffer(x.device).data_ptr(), _lib.stream_ptr())
    _lib.check_rc(rc, "adana_gemm_bf16_gather")
    return out


def linear_fwd_reduce_scatter(x, w, out_ptrs, rows_per_rank: int, me: int, alpha: float = 1.0, ldc=None, push=True):
    """Row-parallel linear fused with its reduce-scatter: this rank's partial product x [M, K_local] · w [N, K_local]ᵀ
    leaves the GEMM epilogue straight for the rank that owns each output row (rank r keeps rows
    [r · rows_per_rank, (r + 1) · rows_per_rank)); `out_ptrs[r]` (tensors or addresses) is rank r's memory, local or
    a peer's over NVLink.
      push=True : bf16 partial rows are STORED into slot `me` of the owner's slot array [n_ranks, rows_per_rank, ldc]
                  (bf16); after a barrier the owner adds its slots with `sum_slots`.  Deterministic, no atomics.
      push=False: fp32 partial rows are ADDED (vector atomics) into the owner's [rows_per_rank, ldc] fp32 buffer, which
                  the owner zeroed (or pre-loaded) before a barrier.
    The caller synchronises the ranks before the call and again before reading.  (The reduce-scatter after
    `RowwiseParallel` in the reference's tensor-parallel plans, src/distributed/fsdp.py:88-103.)"""
    _check2d(x, "x")
    _check2d(w, "w")
    M, K = x.shape
    N = w.shape[0]
    arr, n = _ptr_array(out_ptrs)
    rc = _lib.lib().adana_gemm_bf16_reduce_scatter(
        x.data_ptr(), w.data_ptr(), arr, n, int(me), int(rows_per_rank), M, N, K, x.stride(0), w.stride(0),
        int(ldc if ldc is not None else N), float(alpha), int(bool(push)), _lib.status_buffer(x.device).data_ptr(),
        _lib.stream_ptr())
    _lib.check_rc(rc, "adana_gemm_bf16_reduce_scatter")


def sum_slots(slots, out=None, resid=None, out_lowp=None):
    """out [rows, N] fp32 = (resid or 0) + Σ_s slots[s] (slots [n, rows, N] bf16), fp32 accumulation in slot order;
    `out_lowp` (bf16) optionally receives a copy.  Second half of the push-style reduce-scatter."""
    n, rows, N = slots.shape
    if out is None:
        out = torch.empty((rows, N), dtype=torch.float32, device=slots.device)
    if not (slots.is_cuda and _lib.available()):
        r = slots.float().sum(0) + (0 if resid is None else resid)
        out.copy_(r)
        if out_lowp is not None:
            out_lowp.copy_(r)
        return out
    rc = _lib.lib().adana_sum_slots_bf16(
        slots.data_ptr(), n, rows, N, slots.stride(1), out.data_ptr(), out.stride(0), _lib.ptr(resid),
        0 if resid is None else resid.stride(0), _lib.ptr(out_lowp), 0 if out_lowp is None else out_lowp.stride(0),
        _lib.stream_ptr())
    _lib.check_rc(rc, "adana_sum_slots_bf16")
    return out


def reduce_scatter_partials(partial_ptrs, first_row: int, rows: int, N: int, ld: int, out, resid=None, out_lowp=None):
    """out [rows, N] fp32 = (resid or 0) + Σ_r P_r[first_row : first_row + rows] where rank r's bf16 partial matrix
    P_r (row pitch `ld`) lives at `partial_ptrs[r]` (tensors or addresses; peers are read over NVLink)."""
    arr, n = _ptr_array(partial_ptrs)
    rc = _lib.lib().adana_p2p_reduce_scatter_bf16(
        arr, n, int(first_row), int(rows), int(N), int(ld), out.data_ptr(), out.stride(0), _lib.ptr(resid),
        0 if resid is None else resid.stride(0), _lib.ptr(out_lowp), 0 if out_lowp is None else out_lowp.stride(0),
        _lib.stream_ptr())
    _lib.check_rc(rc, "adana_p2p_reduce_scatter_bf16")
    return out


def linear_fwd_gathered(x, w_shards, rows_per_shard=None, out=None, row_starts=None, me=None, staged=None):
    """y [M, N] = x [M, K] · Wᵀ with W [N, K] split by rows over the shards (equal slices or `row_starts`)."""
    _, n = _ptr_array(w_shards)
    N = row_starts[-1] if row_starts is not None else n * rows_per_shard
    return gather_gemm(x, w_shards, rows_per_shard, N, ldb=x.shape[1], out=out, row_starts=row_starts, me=me,
                       staged=staged)


def linear_gelu_fwd_gathered(x, w_shards, rows_per_shard=None, row_starts=None, me=None, staged=None):
    _, n = _ptr_array(w_shards)
    N = row_starts[-1] if row_starts is not None else n * rows_per_shard
    z = torch.empty((x.shape[0], N), dtype=torch.bfloat16, device=x.device)
    h = torch.empty_like(z)
    gather_gemm(x, w_shards, rows_per_shard, N, ldb=x.shape[1], epi=EPI_GELU_DUAL, out=z, C2=h, row_starts=row_starts,
                me=me, staged=staged)
    return z, h


def linear_dgrad_gathered(dy, w_shards, rows_per_shard, K_out, out=None, row_starts=None, me=None, staged=None):
    """dx [M, K_out] = dy [M, N] · W with W [N, K_out] split by rows (the contraction index is sharded)."""
    return gather_gemm(dy, w_shards, rows_per_shard, K_out, ldb=K_out, b_mn=True, out=out, row_starts=row_starts,
                       me=me, staged=staged)
