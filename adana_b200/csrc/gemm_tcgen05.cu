// Persistent warp-specialised bf16 GEMM for sm_100a:  TMA -> shared memory (128B swizzle)
// -> tcgen05.mma with fp32 accumulators in tensor memory -> fused epilogues.
//
//   D[M,N] = epilogue( A[M,K] * B[N,K]^T )
//
// Operand layouts ("major" = which index is contiguous in global memory):
//   A K-major : memory [M rows][K contiguous]      (activations in a forward pass)
//   A MN-major: memory [K rows][M contiguous]      (dY^T in a weight-gradient GEMM)
//   B K-major : memory [N rows][K contiguous]      (nn.Linear weight [out,in] in forward)
//   B MN-major: memory [K rows][N contiguous]      (weight in dgrad, activations in wgrad)
// so forward, dgrad and wgrad all read the tensors as they are stored; nothing is transposed
// in memory.
//
// CTA = 6 warps: warp 0 issues TMA loads, warp 1 owns tensor memory and issues the MMAs,
// warps 2..5 run the epilogue (each warp reads its own 32-lane quarter of tensor memory).
// Two 256-column accumulators are double-buffered so that the epilogue of tile i overlaps
// the main loop of tile i+1.  Every wait is bounded (see common.cuh).
//
// Replaces the cuBLASLt calls behind nn.Linear in the reference model code
// (src/models/enoki.py:111,150,176-178; src/models/qwen3.py:104-106,173-175,235).
#include <cstdlib>

#include "api.h"
#include "common.cuh"

namespace adana {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int CHUNK_BYTES = BK * 128;  // one 64-wide MN-major chunk: BK rows of 128 B
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;

struct GemmArgs {
  int M, N, K;
  void* C;
  long long ldc;
  void* C2;
  long long ldc2;
  const void* R;
  long long ldr;
  float alpha, beta;
  int b_off2;  // gated-MLP epilogues: offset (rows of B / columns of C,R) of the "up" half
  int tiles_m, tiles_n, group_m;
  int streamk;  // CTA-pair kernel, fp32 output: 0 whole tiles, 1 every K loop cut, 2 only the last wave's
  int* status;
  // EPI_F32_RS (GEMM fused with a reduce-scatter over peers): output rows [r * rs_rows, (r + 1) * rs_rows) are
  // ADDED into rank r's buffer peerC[r] ([rs_rows, ldc] fp32, its own memory or a peer's over NVLink)
  void* peerC[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  int rs_rows = 0;
  int rs_me = 0;  // EPI_BF16_PUSH: this rank's slot in the owner's [n_ranks, rs_rows, ldc] bf16 slot array
  int rot_m = 0;  // row-tile rotation: with it every rank starts on another destination
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int group_m, int& mi,
                                            int& ni) {
  const int per_group = group_m * tiles_n;
  const int g = t / per_group;
  const int first_m = g * group_m;
  const int gm = min(group_m, tiles_m - first_m);
  const int r = t - g * per_group;
  mi = first_m + (r % gm);
  ni = r / gm;
}

// Rows of tiles per raster group.  The tiles that run at the same time (one per CTA or CTA pair) form a block of
// group_m x (concurrency / group_m) tiles; every operand panel is fetched from DRAM once per block that touches it, so
// the operand traffic of a sweep is proportional to 1 / rows + 1 / columns of that block: smallest for a square block,
// and with few tile columns (weight gradients: N / 256 = 9) for a block that spans all of them.
static int pick_group_m(int tiles_m, int tiles_n, int concurrency) {
  static int forced = -1;
  if (forced < 0) {
    const char* e = getenv("ADANA_GEMM_GROUP_M");
    forced = e ? atoi(e) : 0;
  }
  if (forced > 0) return forced;
  int side = 1;
  while ((side + 1) * (side + 1) <= concurrency) ++side;
  if ((side + 1) * (side + 1) - concurrency < concurrency - side * side) ++side;      // nearest square
  const int gn = tiles_n < side ? tiles_n : side;
  int gm = concurrency / (gn > 0 ? gn : 1);
  if (gm < 1) gm = 1;
  if (gm > tiles_m) gm = tiles_m;
  return gm;
}

template <int EPI>
__device__ __forceinline__ void store_bf16x32(__nv_bfloat16* dst, const float (&v)[32], int ncols_ok) {
  // dst is 16-byte aligned (column offsets are multiples of 32, ld multiples of 8)
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (j * 8 < ncols_ok) {
      uint4 q;
      q.x = pack_bf16x2(v[j * 8 + 0], v[j * 8 + 1]);
      q.y = pack_bf16x2(v[j * 8 + 2], v[j * 8 + 3]);
      q.z = pack_bf16x2(v[j * 8 + 4], v[j * 8 + 5]);
      q.w = pack_bf16x2(v[j * 8 + 6], v[j * 8 + 7]);
      *reinterpret_cast<uint4*>(dst + j * 8) = q;
    }
  }
}

__device__ __forceinline__ void load_bf16x32(const __nv_bfloat16* src, float (&v)[32], int ncols_ok) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (j * 8 < ncols_ok) {
      uint4 q = *reinterpret_cast<const uint4*>(src + j * 8);
      float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z),
             d = unpack_bf16x2(q.w);
      v[j * 8 + 0] = a.x; v[j * 8 + 1] = a.y; v[j * 8 + 2] = b.x; v[j * 8 + 3] = b.y;
      v[j * 8 + 4] = c.x; v[j * 8 + 5] = c.y; v[j * 8 + 6] = d.x; v[j * 8 + 7] = d.y;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[j * 8 + i] = 0.f;
    }
  }
}

// One warp's share of a finished accumulator: 32 rows (one per lane) x BN columns read from tensor
// memory at `taddr`, pushed through the epilogue EPI and stored.  `n0` = first output column.
template <int EPI>
__device__ __forceinline__ void epilogue_rows(const GemmArgs& args, uint32_t taddr, int row, bool row_ok,
                                              int n0) {
  if constexpr (EPI == EPI_SWIGLU) {
    // accumulator columns [0,128) = gate, [128,256) = up
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t rg[32], ru[32];
      tmem_ld_32x32b_x32(taddr + c * 32, rg);
      tmem_ld_32x32b_x32(taddr + 128 + c * 32, ru);
      tmem_wait_ld();
      const int col = n0 + c * 32;
      const int ncols_ok = args.N - col;
      if (row_ok && ncols_ok > 0) {
        float g[32], u[32], h[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          g[i] = __uint_as_float(rg[i]);
          u[i] = __uint_as_float(ru[i]);
          h[i] = g[i] * sigmoidf_(g[i]) * u[i];
        }
        __nv_bfloat16* gu = reinterpret_cast<__nv_bfloat16*>(args.C) + (long long)row * args.ldc;
        store_bf16x32<EPI>(gu + col, g, ncols_ok);
        store_bf16x32<EPI>(gu + args.b_off2 + col, u, ncols_ok);
        store_bf16x32<EPI>(reinterpret_cast<__nv_bfloat16*>(args.C2) + (long long)row * args.ldc2 + col,
                           h, ncols_ok);
      }
    }
  } else {
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(taddr + c * 32, r);
      tmem_wait_ld();
      const int col = n0 + c * 32;
      const int ncols_ok = args.N - col;
      if (!row_ok || ncols_ok <= 0) continue;
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * args.alpha;

      if constexpr (EPI == EPI_BF16) {
        store_bf16x32<EPI>(reinterpret_cast<__nv_bfloat16*>(args.C) + (long long)row * args.ldc + col, v,
                           ncols_ok);
      } else if constexpr (EPI == EPI_GELU_DUAL) {
        store_bf16x32<EPI>(reinterpret_cast<__nv_bfloat16*>(args.C) + (long long)row * args.ldc + col, v,
                           ncols_ok);
        float h[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) h[i] = gelu_erf(v[i]);
        store_bf16x32<EPI>(reinterpret_cast<__nv_bfloat16*>(args.C2) + (long long)row * args.ldc2 + col,
                           h, ncols_ok);
      } else if constexpr (EPI == EPI_RESID_F32) {
        const float* rp = reinterpret_cast<const float*>(args.R) + (long long)row * args.ldr + col;
        float* cp = reinterpret_cast<float*>(args.C) + (long long)row * args.ldc + col;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (j * 4 < ncols_ok) {
            float4 x = *reinterpret_cast<const float4*>(rp + j * 4);
            x.x += v[j * 4 + 0];
            x.y += v[j * 4 + 1];
            x.z += v[j * 4 + 2];
            x.w += v[j * 4 + 3];
            *reinterpret_cast<float4*>(cp + j * 4) = x;
          }
        }
      } else if constexpr (EPI == EPI_DGELU) {
        float z[32];
        load_bf16x32(reinterpret_cast<const __nv_bfloat16*>(args.R) + (long long)row * args.ldr + col, z,
                     ncols_ok);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= gelu_erf_grad(z[i]);
        store_bf16x32<EPI>(reinterpret_cast<__nv_bfloat16*>(args.C) + (long long)row * args.ldc + col, v,
                           ncols_ok);
      } else if constexpr (EPI == EPI_AXPBY_BF16) {
        float z[32];
        load_bf16x32(reinterpret_cast<const __nv_bfloat16*>(args.R) + (long long)row * args.ldr + col, z,
                     ncols_ok);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = fmaf(args.beta, z[i], v[i]);
        store_bf16x32<EPI>(reinterpret_cast<__nv_bfloat16*>(args.C) + (long long)row * args.ldc + col, v,
                           ncols_ok);
      } else if constexpr (EPI == EPI_BF16_PUSH) {
        // this rank's partial row goes, with plain stores, into its own slot at the rank that owns the row
        const int owner = row / args.rs_rows;
        __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(args.peerC[owner]) +
                            ((long long)args.rs_me * args.rs_rows + (row - owner * args.rs_rows)) * args.ldc + col;
        store_bf16x32<EPI>(cp, v, ncols_ok);
      } else if constexpr (EPI == EPI_F32_RS) {
        // this rank's partial product of a row that rank `owner` keeps: added in the owner's L2
        const int owner = row / args.rs_rows;
        float* cp = reinterpret_cast<float*>(args.peerC[owner]) + (long long)(row - owner * args.rs_rows) * args.ldc + col;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (j * 4 < ncols_ok)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(cp + j * 4),
                         "f"(v[j * 4]), "f"(v[j * 4 + 1]), "f"(v[j * 4 + 2]), "f"(v[j * 4 + 3])
                         : "memory");
        }
      } else if constexpr (EPI == EPI_F32_ATOMIC) {
        // several CTAs hold partial sums of this tile (split K): add them into C in L2
        float* cp = reinterpret_cast<float*>(args.C) + (long long)row * args.ldc + col;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (j * 4 < ncols_ok)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(cp + j * 4),
                         "f"(v[j * 4]), "f"(v[j * 4 + 1]), "f"(v[j * 4 + 2]), "f"(v[j * 4 + 3])
                         : "memory");
        }
      } else if constexpr (EPI == EPI_F32) {
        float* cp = reinterpret_cast<float*>(args.C) + (long long)row * args.ldc + col;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (j * 4 < ncols_ok) {
            float4 x = make_float4(v[j * 4], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]);
            if (args.beta != 0.f) {
              float4 o = *reinterpret_cast<const float4*>(cp + j * 4);
              x.x += args.beta * o.x;
              x.y += args.beta * o.y;
              x.z += args.beta * o.z;
              x.w += args.beta * o.w;
            }
            *reinterpret_cast<float4*>(cp + j * 4) = x;
          }
        }
      } else if constexpr (EPI == EPI_DSWIGLU) {
        // v = dH chunk; R holds [gate | up] pre-activations, C receives [dGate | dUp]
        const __nv_bfloat16* gu = reinterpret_cast<const __nv_bfloat16*>(args.R) + (long long)row * args.ldr;
        float g[32], u[32];
        load_bf16x32(gu + col, g, ncols_ok);
        load_bf16x32(gu + args.b_off2 + col, u, ncols_ok);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float s = sigmoidf_(g[i]);
          const float dh = v[i];
          const float dgate = dh * u[i] * s * (1.f + g[i] * (1.f - s));
          const float dup = dh * g[i] * s;
          g[i] = dgate;
          u[i] = dup;
        }
        __nv_bfloat16* dgu = reinterpret_cast<__nv_bfloat16*>(args.C) + (long long)row * args.ldc;
        store_bf16x32<EPI>(dgu + col, g, ncols_ok);
        store_bf16x32<EPI>(dgu + args.b_off2 + col, u, ncols_ok);
      } else {
        static_assert(EPI < 0, "epilogue not implemented");
      }
    }
  }
}

template <bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;                 // [STAGES]
  uint64_t* empty_bar = bars + STAGES;       // [STAGES]
  uint64_t* tfull_bar = bars + 2 * STAGES;   // [2]
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr bool GATED_FWD = (EPI == EPI_SWIGLU);
  constexpr int TILE_N = GATED_FWD ? BN / 2 : BN;  // output columns covered by one tile
  const int num_tiles = args.tiles_m * args.tiles_n;
  const int num_kb = (args.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tfull_bar[0], 1);
    mbar_init(&tfull_bar[1], 1);
    mbar_init(&tempty_bar[0], 4);
    mbar_init(&tempty_bar[1], 4);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int mi, ni;
        tile_coords(t, args.tiles_m, args.tiles_n, args.group_m, mi, ni);
        mi += args.rot_m;
        if (mi >= args.tiles_m) mi -= args.tiles_m;
        const int m0 = mi * BM;
        const int n0 = ni * TILE_N;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, args.status,
                         ST_TIMEOUT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sA = smem + stage * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          const int k0 = kb * BK;
          if constexpr (!A_MN) {
            tma_load_2d(sA, &tmA, &full_bar[stage], k0, m0);  // box {64 k, 128 m}
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(sA + c * CHUNK_BYTES, &tmA, &full_bar[stage], m0 + c * 64, k0);
          }
          if constexpr (!B_MN) {
            const int n1 = GATED_FWD ? (args.b_off2 + n0) : (n0 + 128);
            tma_load_2d(sB, &tmB, &full_bar[stage], k0, n0);  // box {64 k, 128 n}
            tma_load_2d(sB + 128 * 128, &tmB, &full_bar[stage], k0, n1);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sB + c * CHUNK_BYTES, &tmB, &full_bar[stage], n0 + c * 64, k0);
          }
          ++issued;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // Aborting: let the copies that are still in flight land before the CTA exits.
        const int pending = issued < STAGES ? (int)issued : STAGES;
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < pending; ++i) {
          if (--s < 0) {
            s = STAGES - 1;
            ph ^= 1;
          }
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&full_bar[s], ph) && globaltimer_ns() - t0 < 20000000ull) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------------
    // The whole warp runs the loop in lock step and one elected lane issues: the descriptors are then computed in
    // warp-uniform code (a tcgen05.mma takes them from uniform registers; inside a one-lane branch every operand of
    // every product is first moved there).  A stage's descriptors are its base descriptor plus the 16-byte-unit
    // offset of the contraction step.
    {
      const bool issuer = elect_one();
      const uint32_t tb = __shfl_sync(0xffffffffu, tmem_base, 0);
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      const uint32_t smem0 = smem_u32(smem);
      const uint64_t a_desc0 = A_MN ? make_smem_desc_sw128(smem0, CHUNK_BYTES, 1024) : make_smem_desc_sw128(smem0, 16, 1024);
      const uint64_t b_desc0 = B_MN ? make_smem_desc_sw128(smem0 + A_BYTES, CHUNK_BYTES, 1024)
                                    : make_smem_desc_sw128(smem0 + A_BYTES, 16, 1024);
      constexpr uint64_t A_STEP = (A_MN ? 2048 : 32) >> 4, B_STEP = (B_MN ? 2048 : 32) >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        const int buf = it & 1;
        const uint32_t use = (uint32_t)(it >> 1);
        if (!mbar_wait_warp(&tempty_bar[buf], (use & 1) ^ 1, abort_flag, args.status, ST_TIMEOUT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tb + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_warp(&full_bar[stage], phase, abort_flag, args.status, ST_TIMEOUT_SMEM_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint64_t da = a_desc0 + (uint64_t)((stage * STAGE_BYTES) >> 4);
          const uint64_t db = b_desc0 + (uint64_t)((stage * STAGE_BYTES) >> 4);
          if (issuer) {
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk)
              umma_ss(tmem_d, da + kk * A_STEP, db + kk * B_STEP, idesc, (kb | kk) != 0 ? 1u : 0u);
            umma_commit(&empty_bar[stage]);  // frees the stage once these MMAs retire
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok && issuer) umma_commit(&tfull_bar[buf]);
      }
    }
  } else {
    // ------------------------------ epilogue (warps 2..5) --------------------------------
    const int quad = warp & 3;  // tensor-memory lane quarter this warp may read
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
      int mi, ni;
      tile_coords(t, args.tiles_m, args.tiles_n, args.group_m, mi, ni);
      mi += args.rot_m;
      if (mi >= args.tiles_m) mi -= args.tiles_m;
      const int buf = it & 1;
      const uint32_t use = (uint32_t)(it >> 1);
      if (!mbar_wait(&tfull_bar[buf], use & 1, abort_flag, args.status, ST_TIMEOUT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int row = mi * BM + quad * 32 + lane;
      const bool row_ok = row < args.M;
      const uint32_t taddr = tmem_base + buf * BN + (uint32_t(quad * 32) << 16);
      const int n0 = ni * TILE_N;

      epilogue_rows<EPI>(args, taddr, row, row_ok, n0);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------
// CTA-pair variant: two CTAs of a cluster (on the two SMs of a TPC) compute one 256 x 256 tile
// with cta_group::2 MMAs.  Each CTA stages only ITS 128 rows of A and ITS 128 of the 256 rows
// (columns) of B, so a k-block costs 32 KiB of shared-memory fill per SM instead of 48 KiB and
// half as many MMA instructions; the accumulator rows [0,128) live in the leader's tensor memory
// and rows [128,256) in the peer's.  Protocol (leader = cluster rank 0):
//   full[s]   on the leader only: one arrive.expect_tx (leader, both CTAs' bytes) + TMA bytes of both
//   empty[s]  in each CTA: one commit per CTA from the leader's MMA thread
//   tfull[b]  in each CTA: one commit per CTA;  tempty[b] on the leader: 8 arrivals (4 epilogue
//   warps of each CTA).  The kernel ends with a cluster barrier so that neither CTA leaves while
//   its partner may still touch its shared memory, barriers or tensor memory.
constexpr int P_STAGES = 7;
constexpr int P_TILE_BYTES = 128 * BK * 2;          // 16 KiB: this CTA's A rows, or its B rows
constexpr int P_STAGE_BYTES = 2 * P_TILE_BYTES;     // 32 KiB
constexpr int P_SMEM = P_STAGES * P_STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int P_BM = 256;

// Work of one CTA pair: whole tiles dealt round-robin, or (stream-K) one contiguous, equal share of
// all (tile, k-block) units cut at tile boundaries into segments; every segment is accumulated from
// zero and added into C by the atomic epilogue, so partial tiles need no fix-up pass.
struct PairWork {
  int tile, kb0, kb1;  // current segment: k-blocks [kb0, kb1) of `tile`
  bool partial;        // the segment is a share of a tile: its result is ADDED into C atomically
  int next_tile, whole_end, step, num_kb;
  long long u, u_end;
  int split_first;
  // mode 0: whole tiles round-robin.  1: every tile's K loop is cut (pure stream-K).
  // 2: the full waves are whole tiles; only the tiles of the last, incomplete wave are cut.
  __device__ PairWork(int pair, int npairs, int num_tiles, int num_kb_, int mode)
      : tile(0), kb0(0), kb1(0), partial(false), next_tile(pair), step(npairs), num_kb(num_kb_) {
    whole_end = mode == 0 ? num_tiles : mode == 1 ? 0 : (num_tiles / npairs) * npairs;
    split_first = whole_end;
    const long long total = (long long)(num_tiles - whole_end) * num_kb;
    u = total * pair / npairs;
    u_end = total * (pair + 1) / npairs;
  }
  __device__ bool next() {
    if (next_tile < whole_end) {
      tile = next_tile;
      kb0 = 0;
      kb1 = num_kb;
      partial = false;
      next_tile += step;
      return true;
    }
    if (u >= u_end) return false;
    const int t = (int)(u / num_kb);
    tile = split_first + t;
    kb0 = (int)(u - (long long)t * num_kb);
    const long long left = u_end - u;
    kb1 = (left < (long long)(num_kb - kb0)) ? kb0 + (int)left : num_kb;
    u += kb1 - kb0;
    partial = true;
    return true;
  }
};

// The B operand of the "gathering" variants: one tensor map per rank over that rank's slice of the
// weight rows (its own memory or a peer's, mapped over NVLink).
//
// Direct variant (SHARDED == 1): the CTA fetches every B box from the rank that owns those rows, so no gathered
// copy of the weight exists.  Peer memory is not cached in the reader's L2, so a remote tile crosses the link once
// per row tile that uses it: right for skinny problems, link-bound for M of many row tiles.
//
// Staged variant (SHARDED == 2): eight extra warps per CTA copy the remote slices, once, with plain 16-byte loads
// from the peers into a local staging matrix, taking 4-row units from a ticket counter in the order in which the
// tiles will want them, and count finished units per chunk (128 weight rows, or one 64-row k-block).  The tile
// order (or the k-loop) is rotated so that work on this rank's own slice comes first; a producer that reaches a
// remote chunk waits (bounded) for its counter, then reads the chunk from the staging matrix with TMA.  Every byte
// of the weight crosses NVLink once and the copy runs under the tiles of the local slice.
constexpr int MAX_SHARDS = 8;
constexpr int GATHER_COPY_WARPS = 8;
constexpr int GATHER_THREADS = GEMM_THREADS + 32 * GATHER_COPY_WARPS;
constexpr int STAGE_UNIT_ROWS = 4;
// Counter layout (ints).  The ticket counter takes an atomic per unit from a thousand warps and the producers poll
// the others, so each of the first two sits on a 128-byte line of its own and the chunk counters are spread one per
// 32-byte sector: polling one chunk does not queue behind the ticket atomics.
constexpr int FLAG_TICKET = 0;
constexpr int FLAG_DONE = 32;
constexpr int FLAG_CHUNK0 = 64;
constexpr int FLAG_CHUNK_STRIDE = 8;
__host__ __device__ constexpr int stage_flag_ints(int nchunks) { return FLAG_CHUNK0 + FLAG_CHUNK_STRIDE * nchunks; }
struct ShardedB {
  CUtensorMap map[MAX_SHARDS];       // 32-row boxes: used where a tile straddles two ranks' slices
  CUtensorMap map_big[MAX_SHARDS];   // whole-tile boxes (128 rows K-major / 64 rows MN-major) for the common case
  CUtensorMap map_stage;             // whole-tile boxes over the staging matrix (rows by their global index)
  const void* ptr[MAX_SHARDS];       // base address of each rank's slice
  void* stage;                 // staging matrix [rows_total, pitch] of this rank
  int* flags;                  // counters, see FLAG_* (ticket, units finished, units finished of chunk c)
  long long pitch_bytes;       // row pitch of the slices and of the staging matrix
  int row_bytes;               // bytes of one weight row (a multiple of 16)
  int rows_total;
  int me;                      // the rank whose slice is local: never staged, never waited for
  int chunk_rows;              // 128 (weight rows = output columns) or 64 (weight rows = contraction index)
  int rot_tile;                // tile (or k-block) rotation that puts the local slice first
  int rot_row;                 // the same in weight rows: where the copy order starts
  int start[MAX_SHARDS + 1];   // rank r holds weight rows [start[r], start[r+1]); every start is a multiple of 32
  int n_shards;
  int use_big;                 // 0 when some slice has fewer rows than a whole-tile box
  __device__ __forceinline__ int owner_of(int row) const {
    int o = 0;
#pragma unroll
    for (int r = 1; r < MAX_SHARDS; ++r) o += (r < n_shards && row >= start[r]) ? 1 : 0;
    return o;
  }
  __device__ __forceinline__ int units_of_chunk(int c) const {
    const int rows = min(chunk_rows, rows_total - c * chunk_rows);
    return (rows + STAGE_UNIT_ROWS - 1) / STAGE_UNIT_ROWS;
  }
  __device__ __forceinline__ int total_units() const {
    return (rows_total + STAGE_UNIT_ROWS - 1) / STAGE_UNIT_ROWS;
  }
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}
__device__ __forceinline__ uint4 ld_peer_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Producer side of the staged variant: has chunk `c` of the staging matrix been filled?  `all_ready` caches the
// answer "every unit is done", after which no counter is read any more.  Bounded like every other wait here.
__device__ __forceinline__ bool stage_wait(const ShardedB* sh, int c, bool& all_ready, bool check_all,
                                           volatile int* abort_flag, int* status) {
  if (all_ready) return true;
  if (check_all && ld_acquire_gpu(sh->flags + FLAG_DONE) >= sh->total_units()) {
    all_ready = true;
    return true;
  }
  const int target = sh->units_of_chunk(c);
  const int* f = sh->flags + FLAG_CHUNK0 + FLAG_CHUNK_STRIDE * c;
  if (ld_acquire_gpu(f) >= target) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (ld_acquire_gpu(f) < target) {
    __nanosleep(200);  // the copier warps need the memory pipes more than this poll does
    if (((++spins) & 0x3fu) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > ADANA_WAIT_TIMEOUT_NS) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, (int)ST_TIMEOUT_PEER_FLAG);
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void copy_vec16(const uint4* __restrict__ src, uint4* __restrict__ dst, int n, int lane) {
  // eight loads in flight per lane (4 KiB per warp), the ragged end predicated rather than serialised
  for (int i = lane; i < n; i += 8 * 32) {
    uint4 t[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (i + j * 32 < n) t[j] = ld_peer_v4(src + i + j * 32);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (i + j * 32 < n) dst[i + j * 32] = t[j];
  }
}

// Copier warps of the staged variant: take 4-row units in rotated row order until none is left.
__device__ __forceinline__ void stage_copy_loop(const ShardedB* sh, int lane) {
  const int total = sh->total_units();
  const int nv = sh->row_bytes >> 4;
  const bool dense = sh->pitch_bytes == (long long)sh->row_bytes;
  int u = 0;
  if (lane == 0) u = atomicAdd(sh->flags + FLAG_TICKET, 1);
  u = __shfl_sync(0xffffffffu, u, 0);
  while (u < total) {
    int next = 0;
    if (lane == 0) next = atomicAdd(sh->flags + FLAG_TICKET, 1);  // the next ticket is on its way while this unit is copied
    int row = u * STAGE_UNIT_ROWS + sh->rot_row;
    if (row >= sh->rows_total) row -= sh->rows_total;
    const int rows = min(STAGE_UNIT_ROWS, sh->rows_total - row);
    const int owner = sh->owner_of(row);
    if (owner != sh->me) {
      const char* src = reinterpret_cast<const char*>(sh->ptr[owner]) + (long long)(row - sh->start[owner]) * sh->pitch_bytes;
      char* dst = reinterpret_cast<char*>(sh->stage) + (long long)row * sh->pitch_bytes;
      if (dense) {
        copy_vec16(reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst), nv * rows, lane);
      } else {
        for (int r = 0; r < rows; ++r)
          copy_vec16(reinterpret_cast<const uint4*>(src + r * sh->pitch_bytes),
                     reinterpret_cast<uint4*>(dst + r * sh->pitch_bytes), nv, lane);
      }
      fence_proxy_async_all();
      __syncwarp();
      if (lane == 0) {
        __threadfence();
        red_release_gpu_add(sh->flags + FLAG_CHUNK0 + FLAG_CHUNK_STRIDE * (row / sh->chunk_rows), 1);
      }
    }
    if (lane == 0) red_release_gpu_add(sh->flags + FLAG_DONE, 1);
    u = __shfl_sync(0xffffffffu, next, 0);
  }
}

template <bool A_MN, bool B_MN, int EPI, int SHARDED>
__device__ __forceinline__ void gemm_pair_body(const CUtensorMap& tmA, const CUtensorMap& tmB,
                                               const ShardedB* __restrict__ shards, const GemmArgs& args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + P_STAGES * P_STAGE_BYTES);
  uint64_t* full_bar = bars;                       // [P_STAGES]  (used on the leader)
  uint64_t* empty_bar = bars + P_STAGES;           // [P_STAGES]
  uint64_t* tfull_bar = bars + 2 * P_STAGES;       // [2]
  uint64_t* tempty_bar = bars + 2 * P_STAGES + 2;  // [2]         (used on the leader)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * P_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int npairs = gridDim.x >> 1;
  constexpr bool GATED_FWD = (EPI == EPI_SWIGLU);
  constexpr int TILE_N = GATED_FWD ? BN / 2 : BN;
  const int num_tiles = args.tiles_m * args.tiles_n;
  const int num_kb = (args.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tfull_bar[0], 1);
    mbar_init(&tfull_bar[1], 1);
    mbar_init(&tempty_bar[0], 8);
    mbar_init(&tempty_bar[1], 8);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the partner's barriers exist before anything remote is sent to them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ---------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      if constexpr (!SHARDED) tma_prefetch_desc(&tmB);
      const uint32_t lead_full0 = mapa_smem(smem_u32(&full_bar[0]), 0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      PairWork w(pair, npairs, num_tiles, num_kb, args.streamk);
      bool all_ready = false;  // staged variant: every remote chunk is known to be in the staging matrix
      // staged variant: what the k-loop needs of the slice table, read once (the copies and waits below are
      // volatile, so nothing read through `shards` inside the loops would stay in a register)
      int loc_lo = 0, loc_hi = 0, st_rot = 0, st_rows = 0, st_chunk = 1;
      const CUtensorMap* map_local = &tmB;
      const CUtensorMap* map_staged = &tmB;
      if constexpr (SHARDED == 2) {
        const int me = shards->me;
        loc_lo = shards->start[me];
        loc_hi = shards->start[me + 1];
        st_rot = shards->rot_tile;
        st_rows = shards->rows_total;
        st_chunk = shards->chunk_rows;
        map_local = &shards->map_big[me];
        map_staged = &shards->map_stage;
      }
      while (ok && w.next()) {
        int mi, ni;
        tile_coords(w.tile, args.tiles_m, args.tiles_n, args.group_m, mi, ni);
        mi += args.rot_m;
        if (mi >= args.tiles_m) mi -= args.tiles_m;
        if constexpr (SHARDED == 2 && !B_MN) {  // tiles on this rank's own slice first
          ni += st_rot;
          if (ni >= args.tiles_n) ni -= args.tiles_n;
        }
        const int m0 = mi * P_BM + (int)rank * 128;  // this CTA's rows of A and of the output
        const int n0 = ni * TILE_N;
        // this CTA's 128 rows (columns) of B: second half of the tile, or the "up" rows when gated
        const int nb0 = GATED_FWD ? (leader ? n0 : args.b_off2 + n0) : n0 + (int)rank * 128;
        bool b_staged = false;  // staged variant, weight rows = output columns: one owner per tile half
        if constexpr (SHARDED == 2 && !B_MN) {
          b_staged = nb0 < loc_lo || nb0 >= loc_hi;
          if (b_staged && nb0 < st_rows &&
              !stage_wait(shards, nb0 / st_chunk, all_ready, true, abort_flag, args.status)) {
            ok = false;
            break;
          }
        }
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          int kbr = kb;
          if constexpr (SHARDED == 2 && B_MN) {  // the k-loop starts on this rank's own slice
            kbr += st_rot;
            if (kbr >= num_kb) kbr -= num_kb;
            const int kr = kbr * BK;
            b_staged = kr < loc_lo || kr >= loc_hi;
            if (b_staged && kr < st_rows &&
                !stage_wait(shards, kbr, all_ready, ((kb - w.kb0) & 7) == 0, abort_flag, args.status)) {
              ok = false;
              break;
            }
          }
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, args.status,
                         ST_TIMEOUT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sA = smem + stage * P_STAGE_BYTES;
          uint8_t* sB = sA + P_TILE_BYTES;
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * P_STAGE_BYTES);
          const uint32_t bar = lead_full0 + stage * 8;
          const int k0 = kbr * BK;
          if constexpr (!A_MN) {
            tma_load_2d_pair(sA, &tmA, bar, k0, m0);  // box {64 k, 128 m}
          } else {
#pragma unroll
            for (int c = 0; c < 2; ++c)
              tma_load_2d_pair(sA + c * CHUNK_BYTES, &tmA, bar, m0 + c * 64, k0);
          }
          if constexpr (SHARDED == 2) {
            // slices are cut on whole chunks here: the local slice is read in place, the rest from staging
            const CUtensorMap* mp = b_staged ? map_staged : map_local;
            const int off = b_staged ? 0 : loc_lo;
            if constexpr (!B_MN) {
              tma_load_2d_pair(sB, mp, bar, k0, nb0 - off);
            } else {
#pragma unroll
              for (int c = 0; c < 2; ++c) tma_load_2d_pair(sB + c * CHUNK_BYTES, mp, bar, nb0 + c * 64, k0 - off);
            }
          } else if constexpr (SHARDED == 1) {
            if constexpr (!B_MN) {
              // weight rows = output columns.  One {64 k, 128 n} box when the 128 rows belong to one rank,
              // else 4 boxes {64 k, 32 n}, each from the rank owning those rows
              const int o_lo = shards->owner_of(nb0), o_hi = shards->owner_of(nb0 + 127);
              if (o_lo == o_hi && shards->use_big) {
                tma_load_2d_pair(sB, &shards->map_big[o_lo], bar, k0, nb0 - shards->start[o_lo]);
              } else {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const int row = nb0 + q * 32;
                  const int owner = shards->owner_of(row);
                  tma_load_2d_pair(sB + q * 32 * 128, &shards->map[owner], bar, k0, row - shards->start[owner]);
                }
              }
            } else {
              // weight rows = the contraction index: {64 n, 64 k} boxes per 64-column chunk, or two
              // {64 n, 32 k} boxes where the k-block straddles two ranks
              const int o_lo = shards->owner_of(k0), o_hi = shards->owner_of(k0 + 63);
              if (o_lo == o_hi && shards->use_big) {
#pragma unroll
                for (int c = 0; c < 2; ++c)
                  tma_load_2d_pair(sB + c * CHUNK_BYTES, &shards->map_big[o_lo], bar, nb0 + c * 64,
                                   k0 - shards->start[o_lo]);
              } else {
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                  const int row = k0 + q * 32;
                  const int owner = shards->owner_of(row);
#pragma unroll
                  for (int c = 0; c < 2; ++c)
                    tma_load_2d_pair(sB + c * CHUNK_BYTES + q * 32 * 128, &shards->map[owner], bar, nb0 + c * 64,
                                     row - shards->start[owner]);
                }
              }
            }
          } else if constexpr (!B_MN) {
            tma_load_2d_pair(sB, &tmB, bar, k0, nb0);  // box {64 k, 128 n}
          } else {
#pragma unroll
            for (int c = 0; c < 2; ++c)
              tma_load_2d_pair(sB + c * CHUNK_BYTES, &tmB, bar, nb0 + c * 64, k0);
          }
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // Aborting: copies still in flight land within microseconds; give them a millisecond
        // before this CTA heads for the final cluster barrier.
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 1000000ull) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) -------------------------
    // Warp-uniform loop with one elected issuing lane (see the one-CTA kernel above).
    if (leader) {
      const bool issuer = elect_one();
      const uint32_t tb = __shfl_sync(0xffffffffu, tmem_base, 0);
      constexpr uint32_t idesc = make_idesc_bf16(P_BM, BN, A_MN, B_MN);
      const uint32_t own_empty0 = smem_u32(&empty_bar[0]);
      const uint32_t peer_empty0 = mapa_smem(own_empty0, 1);
      const uint32_t own_tfull0 = smem_u32(&tfull_bar[0]);
      const uint32_t peer_tfull0 = mapa_smem(own_tfull0, 1);
      const uint32_t smem0 = smem_u32(smem);
      const uint64_t a_desc0 = A_MN ? make_smem_desc_sw128(smem0, CHUNK_BYTES, 1024) : make_smem_desc_sw128(smem0, 16, 1024);
      const uint64_t b_desc0 = B_MN ? make_smem_desc_sw128(smem0 + P_TILE_BYTES, CHUNK_BYTES, 1024)
                                    : make_smem_desc_sw128(smem0 + P_TILE_BYTES, 16, 1024);
      constexpr uint64_t A_STEP = (A_MN ? 2048 : 32) >> 4, B_STEP = (B_MN ? 2048 : 32) >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      PairWork w(pair, npairs, num_tiles, num_kb, args.streamk);
      for (; ok && w.next(); ++it) {
        const int buf = it & 1;
        const uint32_t use = (uint32_t)(it >> 1);
        if (!mbar_wait_warp(&tempty_bar[buf], (use & 1) ^ 1, abort_flag, args.status, ST_TIMEOUT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tb + buf * BN;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait_warp(&full_bar[stage], phase, abort_flag, args.status, ST_TIMEOUT_SMEM_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint64_t da = a_desc0 + (uint64_t)((stage * P_STAGE_BYTES) >> 4);
          const uint64_t db = b_desc0 + (uint64_t)((stage * P_STAGE_BYTES) >> 4);
          if (issuer) {
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk)
              umma_ss_pair(tmem_d, da + kk * A_STEP, db + kk * B_STEP, idesc, (kb != w.kb0 || kk != 0) ? 1u : 0u);
            // the stage is free in BOTH CTAs once these MMAs retire
            umma_commit_pair(own_empty0 + stage * 8);
            umma_commit_pair(peer_empty0 + stage * 8);
          }
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok && issuer) {
          umma_commit_pair(own_tfull0 + buf * 8);
          umma_commit_pair(peer_tfull0 + buf * 8);
        }
      }
    }
  } else if (warp >= GEMM_THREADS / 32) {
    // ------------------------------ copier warps (staged variant only) -----------------------
    if constexpr (SHARDED == 2) stage_copy_loop(shards, lane);
  } else {
    // ------------------------------ epilogue (warps 2..5 of both CTAs) -----------------------
    const int quad = warp & 3;
    const uint32_t lead_tempty0 = mapa_smem(smem_u32(&tempty_bar[0]), 0);
    int it = 0;
    bool ok = true;
    PairWork w(pair, npairs, num_tiles, num_kb, args.streamk);
    for (; ok && w.next(); ++it) {
      int mi, ni;
      tile_coords(w.tile, args.tiles_m, args.tiles_n, args.group_m, mi, ni);
      mi += args.rot_m;
      if (mi >= args.tiles_m) mi -= args.tiles_m;
      if constexpr (SHARDED == 2 && !B_MN) {
        ni += shards->rot_tile;
        if (ni >= args.tiles_n) ni -= args.tiles_n;
      }
      const int buf = it & 1;
      const uint32_t use = (uint32_t)(it >> 1);
      if (!mbar_wait(&tfull_bar[buf], use & 1, abort_flag, args.status, ST_TIMEOUT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int row = mi * P_BM + (int)rank * 128 + quad * 32 + lane;
      const bool row_ok = row < args.M;
      const uint32_t taddr = tmem_base + buf * BN + (uint32_t(quad * 32) << 16);
      if constexpr (EPI == EPI_F32) {
        if (w.partial) epilogue_rows<EPI_F32_ATOMIC>(args, taddr, row, row_ok, ni * TILE_N);
        else epilogue_rows<EPI_F32>(args, taddr, row, row_ok, ni * TILE_N);
      } else {
        epilogue_rows<EPI>(args, taddr, row, row_ok, ni * TILE_N);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(lead_tempty0 + buf * 8);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

template <bool A_MN, bool B_MN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const GemmArgs args) {
  gemm_pair_body<A_MN, B_MN, EPI, 0>(tmA, tmB, nullptr, args);
}

// All-gather fused into the GEMM: B is read shard by shard from the ranks that own it.
template <bool B_MN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_gather_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ ShardedB shards,
                        const GemmArgs args) {
  gemm_pair_body<false, B_MN, EPI, 1>(tmA, shards.map[0], &shards, args);
}

// The same with every remote slice brought over the link once (see ShardedB).
template <bool B_MN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GATHER_THREADS, 1)
gemm_bf16_gather_staged_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ ShardedB shards,
                               const GemmArgs args) {
  gemm_pair_body<false, B_MN, EPI, 2>(tmA, shards.map[0], &shards, args);
}

// ------------------------------------------------------------------------------------------------
template <bool A_MN, bool B_MN, int EPI>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& args,
                       int sm_count, cudaStream_t stream) {
  auto kern = gemm_bf16_kernel<A_MN, B_MN, EPI>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = args.tiles_m * args.tiles_n;
  const int grid = tiles < sm_count ? tiles : sm_count;
  kern<<<grid, GEMM_THREADS, GEMM_SMEM, stream>>>(tmA, tmB, args);
  return (int)cudaGetLastError();
}

template <bool A_MN, bool B_MN, int EPI>
static int launch_gemm_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmArgs args, int sm_count,
                            cudaStream_t stream) {
  auto kern = gemm_bf16_pair_kernel<A_MN, B_MN, EPI>;
  static int max_pairs = 0;  // co-resident CTA pairs, asked once per instantiation
  if (max_pairs == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((sm_count / 2) * 2);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = P_SMEM;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    if (e != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count / 2;
    }
    max_pairs = n < sm_count / 2 ? n : sm_count / 2;
  }
  args.tiles_m = (args.M + P_BM - 1) / P_BM;
  const int tiles = args.tiles_m * args.tiles_n;
  int pairs = tiles < max_pairs ? tiles : max_pairs;
  if (args.streamk) {
    const long long units = (long long)tiles * ((args.K + BK - 1) / BK);
    pairs = units < max_pairs ? (int)units : max_pairs;
  }
  kern<<<2 * pairs, GEMM_THREADS, P_SMEM, stream>>>(tmA, tmB, args);
  return (int)cudaGetLastError();
}

template <bool B_MN, int EPI, bool STAGED>
static int launch_gemm_gather_impl(const CUtensorMap& tmA, const ShardedB& shards, GemmArgs args, int sm_count,
                                   cudaStream_t stream) {
  auto kern = STAGED ? gemm_bf16_gather_staged_kernel<B_MN, EPI> : gemm_bf16_gather_kernel<B_MN, EPI>;
  constexpr int threads = STAGED ? GATHER_THREADS : GEMM_THREADS;
  static int max_pairs = 0;
  if (max_pairs == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((sm_count / 2) * 2);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = P_SMEM;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    if (e != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count / 2;
    }
    max_pairs = n < sm_count / 2 ? n : sm_count / 2;
  }
  args.tiles_m = (args.M + P_BM - 1) / P_BM;
  const int tiles = args.tiles_m * args.tiles_n;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  if (STAGED) {
    const int nchunks = (shards.rows_total + shards.chunk_rows - 1) / shards.chunk_rows;
    cudaError_t e = cudaMemsetAsync(shards.flags, 0, sizeof(int) * stage_flag_ints(nchunks), stream);
    if (e != cudaSuccess) return (int)e;
  }
  kern<<<2 * pairs, threads, P_SMEM, stream>>>(tmA, shards, args);
  return (int)cudaGetLastError();
}

template <bool B_MN, int EPI>
static int launch_gemm_gather(const CUtensorMap& tmA, const ShardedB& shards, const GemmArgs& args, int sm_count,
                              cudaStream_t stream) {
  return shards.stage ? launch_gemm_gather_impl<B_MN, EPI, true>(tmA, shards, args, sm_count, stream)
                      : launch_gemm_gather_impl<B_MN, EPI, false>(tmA, shards, args, sm_count, stream);
}

static int g_sm_count = 0;
static int g_gemm_mode = 0;  // 0: per shape, 1: single-CTA tiles, 2: CTA-pair tiles (+stream-K), 3: pair, no stream-K

}  // namespace adana

using namespace adana;

extern "C" int adana_gemm_set_mode(int mode) {
  const int old = g_gemm_mode;
  if (mode >= 0 && mode <= 3) g_gemm_mode = mode;
  return old;
}

extern "C" int adana_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K,
                               long long lda, long long ldb, long long ldc, int a_mn, int b_mn,
                               int epi, void* C2, long long ldc2, const void* R, long long ldr,
                               float alpha, float beta, int b_off2, int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N % 8) != 0 || (ldc % 4) != 0) return -100;
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap tmA, tmB;
  int rc;
  if (!a_mn)
    rc = encode_tmap_2d(&tmA, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 64, BM, 2);
  else
    rc = encode_tmap_2d(&tmA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, BK, 2);
  if (rc) return -101;
  const bool gated_fwd = (epi == EPI_SWIGLU);
  // B holds N rows (K-major) or N columns (MN-major); the gated forward reads 2*N of them.
  const uint64_t b_extent = gated_fwd ? (uint64_t)(b_off2 + N) : (uint64_t)N;
  if (!b_mn)
    rc = encode_tmap_2d(&tmB, B, (uint64_t)K, b_extent, (uint64_t)ldb, 64, 128, 2);
  else
    rc = encode_tmap_2d(&tmB, B, b_extent, (uint64_t)K, (uint64_t)ldb, 64, BK, 2);
  if (rc) return -102;

  GemmArgs args;
  args.M = M; args.N = N; args.K = K;
  args.C = C; args.ldc = ldc; args.C2 = C2; args.ldc2 = ldc2; args.R = R; args.ldr = ldr;
  args.alpha = alpha; args.beta = beta; args.b_off2 = b_off2;
  args.tiles_m = (M + BM - 1) / BM;
  const int tile_n = gated_fwd ? BN / 2 : BN;
  args.tiles_n = (N + tile_n - 1) / tile_n;
  args.group_m = 16;
  args.status = status;

  // CTA-pair tiles are 256 rows tall: worth it when the pairs still get at least ~2 full waves.
  const long long pair_tiles = (long long)((M + P_BM - 1) / P_BM) * args.tiles_n;
  const int npairs = g_sm_count / 2;
  bool use_pair = g_gemm_mode >= 2;
  if (g_gemm_mode == 0) use_pair = pair_tiles >= 2 * npairs || (epi == EPI_F32 && pair_tiles >= npairs);
  // fp32 accumulate-or-overwrite outputs (weight gradients: few tiles, long K).  Whole tiles leave
  // the machine idle in the last wave (243 tiles on 74 pairs: a fourth wave for 21 tiles).  Cutting
  // EVERY K loop and adding partial tiles atomically (mode 2) costs more in fp32 vector atomics than
  // it saves (measured 0.56 ms against 0.41 ms for the 16384x6912x2304 weight gradient), so the
  // per-shape policy cuts only the tiles of that last, incomplete wave: the full waves store
  // normally and at most one atomic partial per pair is added.
  args.streamk = 0;
  if (epi == EPI_F32 && (beta == 0.f || beta == 1.f) && use_pair && (K + BK - 1) / BK >= 8 &&
      (g_gemm_mode == 0 || g_gemm_mode == 2)) {
    const long long rem = pair_tiles % npairs;
    const bool tail_idle = rem != 0 && rem * 10 < npairs * 9;
    if (g_gemm_mode == 2 || tail_idle) {
      args.streamk = g_gemm_mode == 2 ? 1 : 2;
      if (beta == 0.f) {
        // partial tiles are added, not stored: start them from zero
        cudaError_t e = cudaMemset2DAsync(C, (size_t)ldc * 4, 0, (size_t)N * 4, (size_t)M, stream);
        if (e != cudaSuccess) return (int)e;
        args.beta = 0.f;
      }
    }
  }
  args.group_m = pick_group_m(use_pair ? (M + P_BM - 1) / P_BM : args.tiles_m, args.tiles_n,
                              use_pair ? g_sm_count / 2 : g_sm_count);
#define ADANA_GEMM_CASE(AM, BMN, E)                                                     \
  if (a_mn == (AM ? 1 : 0) && b_mn == (BMN ? 1 : 0) && epi == E)                        \
    return use_pair ? launch_gemm_pair<AM, BMN, E>(tmA, tmB, args, g_sm_count, stream)  \
                    : launch_gemm<AM, BMN, E>(tmA, tmB, args, g_sm_count, stream);
  // forward (activations x weight^T)
  ADANA_GEMM_CASE(false, false, EPI_BF16)
  ADANA_GEMM_CASE(false, false, EPI_GELU_DUAL)
  ADANA_GEMM_CASE(false, false, EPI_RESID_F32)
  ADANA_GEMM_CASE(false, false, EPI_F32)
  ADANA_GEMM_CASE(false, false, EPI_SWIGLU)
  ADANA_GEMM_CASE(false, false, EPI_AXPBY_BF16)
  // dgrad (dY x weight)
  ADANA_GEMM_CASE(false, true, EPI_BF16)
  ADANA_GEMM_CASE(false, true, EPI_DGELU)
  ADANA_GEMM_CASE(false, true, EPI_DSWIGLU)
  ADANA_GEMM_CASE(false, true, EPI_F32)
  ADANA_GEMM_CASE(false, true, EPI_RESID_F32)
  ADANA_GEMM_CASE(false, true, EPI_AXPBY_BF16)
  // wgrad (dY^T x X)
  ADANA_GEMM_CASE(true, true, EPI_F32)
  ADANA_GEMM_CASE(true, true, EPI_BF16)
  // generic extras
  ADANA_GEMM_CASE(true, false, EPI_BF16)
  ADANA_GEMM_CASE(true, false, EPI_F32)
#undef ADANA_GEMM_CASE
  return -103;
}

extern "C" int adana_gemm_bf16_reduce_scatter(const void* A, const void* B, void* const* C_ranks, int n_ranks,
                                              int my_rank, int rows_per_rank, int M, int N, int K, long long lda,
                                              long long ldb, long long ldc, float alpha, int push_bf16,
                                              int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (n_ranks < 1 || n_ranks > 8 || my_rank < 0 || my_rank >= n_ranks || rows_per_rank <= 0) return -110;
  if (push_bf16 && (ldc % 8) != 0) return -100;
  if ((long long)rows_per_rank * n_ranks < M) return -111;
  if ((N % 8) != 0 || (ldc % 4) != 0) return -100;
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap tmA, tmB;
  if (encode_tmap_2d(&tmA, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 64, BM, 2)) return -101;
  if (encode_tmap_2d(&tmB, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 64, 128, 2)) return -102;
  GemmArgs args;
  args.M = M; args.N = N; args.K = K;
  args.C = nullptr; args.ldc = ldc; args.C2 = nullptr; args.ldc2 = 0; args.R = nullptr; args.ldr = 0;
  args.alpha = alpha; args.beta = 0.f; args.b_off2 = 0;
  args.tiles_n = (N + BN - 1) / BN;
  args.group_m = 16;
  args.streamk = 0;
  args.status = status;
  for (int r = 0; r < 8; ++r) {
    args.peerC[r] = C_ranks[r < n_ranks ? r : 0];
    if ((reinterpret_cast<uintptr_t>(args.peerC[r]) % 16) != 0) return -100;
  }
  args.rs_rows = rows_per_rank;
  args.rs_me = my_rank;
  const long long pair_tiles = (long long)((M + P_BM - 1) / P_BM) * args.tiles_n;
  const bool use_pair = g_gemm_mode >= 2 || (g_gemm_mode == 0 && pair_tiles >= 2 * (g_sm_count / 2));
  const int tile_rows = use_pair ? P_BM : BM;
  args.tiles_m = (M + tile_rows - 1) / tile_rows;
  // first row tile of the next rank's rows
  args.rot_m = (int)(((long long)((my_rank + 1) % n_ranks) * rows_per_rank / tile_rows) % args.tiles_m);
  if (push_bf16)
    return use_pair ? launch_gemm_pair<false, false, EPI_BF16_PUSH>(tmA, tmB, args, g_sm_count, stream)
                    : launch_gemm<false, false, EPI_BF16_PUSH>(tmA, tmB, args, g_sm_count, stream);
  return use_pair ? launch_gemm_pair<false, false, EPI_F32_RS>(tmA, tmB, args, g_sm_count, stream)
                  : launch_gemm<false, false, EPI_F32_RS>(tmA, tmB, args, g_sm_count, stream);
}

// C = epilogue(A * W^T) (b_mn = 0, W [N, K] split by rows over the ranks) or C = epilogue(A * W) (b_mn = 1,
// W [K, N] split by rows), where rank r holds rows [row_starts[r], row_starts[r+1]) of W at B_shards[r] (this rank's
// memory or a peer's) with row pitch ldb; every start is a multiple of 32.  row_starts == nullptr: equal slices
// of rows_per_shard rows.  Slices cut on multiples of 128 rows (64 for b_mn = 1) are fetched with whole-tile boxes
// only.  stage == nullptr: every B box is fetched from its owner each time it is used, nothing is staged.
// stage != nullptr (a [rows of W, ldb] bf16 matrix of this rank) with flags (64 + rows / 8 ints) and my_rank: the
// remote slices are copied into `stage` once, inside the same kernel, while the tiles on my_rank's own slice run;
// needs every slice cut on multiples of 128 rows (64 for b_mn = 1).  Launches that share `stage` and `flags` must
// be ordered on one stream.
extern "C" int adana_gemm_bf16_gather(const void* A, const void* const* B_shards, int n_shards,
                                      int rows_per_shard, const int* row_starts, void* C, int M, int N, int K,
                                      long long lda, long long ldb, long long ldc, int b_mn, int epi, void* C2,
                                      long long ldc2, const void* R, long long ldr, float alpha, int my_rank,
                                      void* stage, int* flags, int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (n_shards < 1 || n_shards > MAX_SHARDS) return -110;
  if ((N % 8) != 0 || (ldc % 4) != 0) return -100;
  ShardedB sh;
  sh.n_shards = n_shards;
  for (int r = 0; r <= MAX_SHARDS; ++r) {
    const int rr = r < n_shards ? r : n_shards;
    sh.start[r] = row_starts ? row_starts[rr] : rr * rows_per_shard;
  }
  const uint32_t big_rows = b_mn ? 64 : 128;
  sh.use_big = 1;
  for (int r = 0; r < n_shards; ++r) {
    const int rows = sh.start[r + 1] - sh.start[r];
    if (rows <= 0 || (rows % 32) != 0 || (sh.start[r] % 32) != 0) return -110;
    if (rows < (int)big_rows) sh.use_big = 0;
  }
  if (sh.start[0] != 0 || sh.start[n_shards] < (b_mn ? K : N)) return -111;
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap tmA;
  if (encode_tmap_2d(&tmA, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 64, BM, 2)) return -101;
  for (int r = 0; r < n_shards; ++r) {
    const uint64_t inner = b_mn ? (uint64_t)N : (uint64_t)K;
    const uint64_t rows = (uint64_t)(sh.start[r + 1] - sh.start[r]);
    if (encode_tmap_2d(&sh.map[r], B_shards[r], inner, rows, (uint64_t)ldb, 64, 32, 2)) return -102;
    if (encode_tmap_2d(&sh.map_big[r], B_shards[r], inner, rows, (uint64_t)ldb, 64, sh.use_big ? big_rows : 32, 2))
      return -102;
  }
  for (int r = n_shards; r < MAX_SHARDS; ++r) {
    sh.map[r] = sh.map[0];
    sh.map_big[r] = sh.map_big[0];
  }
  for (int r = 0; r < MAX_SHARDS; ++r) sh.ptr[r] = B_shards[r < n_shards ? r : 0];
  sh.map_stage = sh.map_big[0];
  sh.stage = nullptr;
  sh.flags = flags;
  sh.pitch_bytes = ldb * 2;
  sh.row_bytes = (b_mn ? N : K) * 2;
  sh.rows_total = b_mn ? K : N;
  sh.me = my_rank;
  sh.chunk_rows = (int)big_rows;
  sh.rot_tile = 0;
  sh.rot_row = 0;
  if (stage != nullptr) {
    if (flags == nullptr || my_rank < 0 || my_rank >= n_shards || !sh.use_big) return -112;
    if ((sh.row_bytes % 16) != 0 || (sh.pitch_bytes % 16) != 0 || (reinterpret_cast<uintptr_t>(stage) % 16) != 0)
      return -112;
    for (int r = 0; r < n_shards; ++r) {
      if ((sh.start[r] % (int)big_rows) != 0) return -112;
      if ((reinterpret_cast<uintptr_t>(B_shards[r]) % 16) != 0) return -112;
    }
    if (sh.start[n_shards] != sh.rows_total) return -112;
    sh.stage = stage;
    const uint64_t inner = b_mn ? (uint64_t)N : (uint64_t)K;
    if (encode_tmap_2d(&sh.map_stage, stage, inner, (uint64_t)sh.rows_total, (uint64_t)ldb, 64, big_rows, 2))
      return -102;
    if (!b_mn) {
      // first whole tile of the local slice; a tile that straddles the slice's start goes last, with the
      // neighbour's rows that are copied last
      const int tiles_n = (N + BN - 1) / BN;
      sh.rot_tile = ((sh.start[my_rank] + BN - 1) / BN) % tiles_n;
      sh.rot_row = sh.rot_tile * BN >= sh.rows_total ? 0 : sh.rot_tile * BN;
    } else {
      sh.rot_tile = sh.start[my_rank] / BK;
      sh.rot_row = sh.start[my_rank];
    }
  }
  GemmArgs args;
  args.M = M; args.N = N; args.K = K;
  args.C = C; args.ldc = ldc; args.C2 = C2; args.ldc2 = ldc2; args.R = R; args.ldr = ldr;
  args.alpha = alpha; args.beta = 0.f; args.b_off2 = 0;
  args.tiles_m = (M + P_BM - 1) / P_BM;
  args.tiles_n = (N + BN - 1) / BN;
  args.group_m = 16;
  args.streamk = 0;
  args.status = status;
  if (!b_mn && epi == EPI_BF16) return launch_gemm_gather<false, EPI_BF16>(tmA, sh, args, g_sm_count, stream);
  if (!b_mn && epi == EPI_GELU_DUAL) return launch_gemm_gather<false, EPI_GELU_DUAL>(tmA, sh, args, g_sm_count, stream);
  if (!b_mn && epi == EPI_RESID_F32) return launch_gemm_gather<false, EPI_RESID_F32>(tmA, sh, args, g_sm_count, stream);
  if (b_mn && epi == EPI_BF16) return launch_gemm_gather<true, EPI_BF16>(tmA, sh, args, g_sm_count, stream);
  if (b_mn && epi == EPI_DGELU) return launch_gemm_gather<true, EPI_DGELU>(tmA, sh, args, g_sm_count, stream);
  return -103;
}

ADANA_DBG_BIND(gemm)
