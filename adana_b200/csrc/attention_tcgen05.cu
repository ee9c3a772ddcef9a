// Causal self-attention forward on tcgen05 tensor cores (sm_100a), head_dim 64 or 128, bf16.
//
// One CTA = one (batch, head, 128-query tile); it walks the key/value tiles 0..diagonal:
//   warp 0      TMA producer: Q once, then K_j / V_j tiles through a 2-stage ring (128B swizzle)
//   warp 1      MMA issuer:  S_j = Q K_j^T  -> tensor memory          (both operands K-major)
//                            O  += P_j V_j  -> tensor memory          (P K-major, V MN-major)
//   warps 2..5  softmax: thread r owns query row r (tcgen05.ld 32x32b gives one row per lane, so the
//               row max / row sum need no shuffles), writes P_j as bf16 into shared memory in the
//               128B-swizzled K-major layout the MMA reads, rescales O in tensor memory lazily (only
//               when the running max grew by more than 2^8), and finally normalises and stores O.
// With head_dim 128 one CTA fills an SM and four softmax warps (one per scheduler) cannot keep the exponential unit
// busy, so there eight warps do the softmax (SW = 8): two per 32 rows, each taking 64 of the tile's 128 key columns;
// the pair agrees on the row maximum through shared memory (one 64-thread named barrier per tile) and shares the
// rescaling of O, the P store and the epilogue by columns.
// QK_{j+1} is issued before PV_j waits for P_j, so the tensor cores compute the next scores while
// the softmax of the current tile runs; with head_dim 64 two CTAs share an SM and overlap each other.
// Grouped-query attention: query head h reads KV head h / (Hq/Hk).  V is read in place from the fused
// projection output through a strided tensor map.  Every wait is bounded (common.cuh).
//
// Also writes lse2[b, h, s] = log2(sum_j exp(scale * s_ij)) in log2 units, which the backward uses
// to recompute P without a second pass over the row.
//
// Replaces F.scaled_dot_product_attention(is_causal=True) of the reference
// (src/models/enoki.py:134-136, src/models/qwen3.py:212-217).
#include <cstdlib>

#include "api.h"
#include "common.cuh"

namespace adana {

constexpr int ATT_BQ = 128;
constexpr int ATT_BKV = 128;
constexpr int ATT_BWD_THREADS = 448;   // TMA warp, MMA warp, eight score warps (two per lane quarter), four dQ drain warps
constexpr int ATT_KV_STAGES = 2;
constexpr float ATT_RESCALE_THRESHOLD = 8.0f;  // log2 units

template <int HD>
struct AttFwdSmem {
  static constexpr int TILE = ATT_BQ * HD * 2;            // one [128, HD] bf16 tile
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = TILE;
  static constexpr int V_OFF = K_OFF + ATT_KV_STAGES * TILE;
  static constexpr int BAR_OFF = V_OFF + ATT_KV_STAGES * TILE;
  static constexpr int TOTAL = BAR_OFF + 256;              // + barriers (the base is 1024-byte aligned)
};

struct AttFwdArgs {
  __nv_bfloat16* out;     // [T, Hq*HD]
  float* lse2;            // [B, Hq, S]
  int B, S, Hq, Hk;
  float scale_log2;       // softmax scale * log2(e)
  int* status;
};

// 64-thread barrier of the two softmax warps that share 32 rows; the id is an immediate so that the kernel reserves
// five barriers, not all sixteen
__device__ __forceinline__ void pair_barrier(int quad) {
  switch (quad) {
    case 0: named_barrier_sync(1, 64); break;
    case 1: named_barrier_sync(2, 64); break;
    case 2: named_barrier_sync(3, 64); break;
    default: named_barrier_sync(4, 64); break;
  }
}

template <int HD, int S_BUFS, int SW>
__global__ void __launch_bounds__(64 + 32 * SW, (HD == 64 ? 2 : 1))
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttFwdArgs args) {
  using L = AttFwdSmem<HD>;
  constexpr int CHUNKS = HD / 64;                 // 64-column (128-byte) chunks per tile row
  constexpr int CHUNK_BYTES = ATT_BQ * 128;       // [128 rows][128 B]
  // tensor memory columns: S buffers | O accumulator | P (bf16 pairs: 64 columns for 128 keys)
  constexpr uint32_t O_COL = S_BUFS * 128;
  constexpr uint32_t P_COL = O_COL + HD;
  constexpr uint32_t TMEM_COLS = (P_COL + ATT_BKV / 2) <= 256 ? 256 : 512;

  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* q_full = bars;                 // [1]
  uint64_t* k_full = bars + 1;             // [STAGES]
  uint64_t* v_full = bars + 3;             // [STAGES]
  uint64_t* k_empty = bars + 5;            // [STAGES]  K_j is free once QK_j has run ...
  uint64_t* v_empty = bars + 14;           // [STAGES]  ... V_j only after PV_j: K_{j+2} is fetched a whole tile earlier
  uint64_t* s_full = bars + 7;             // [2]
  uint64_t* s_empty = bars + 9;            // [2]
  uint64_t* p_full = bars + 11;            // [1]
  uint64_t* p_empty = bars + 12;           // [1]
  uint64_t* o_full = bars + 13;            // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = args.S / ATT_BQ;
  const int BH = args.B * args.Hq;
  // heaviest query tiles (most KV tiles) are scheduled first
  const int qt = n_qt - 1 - (int)(blockIdx.x / BH);
  const int bh = (int)(blockIdx.x % BH);
  const int b = bh / args.Hq, h = bh % args.Hq;
  const int hk = h / (args.Hq / args.Hk);
  const int n_kv = qt + 1;
  const int row0 = b * args.S + qt * ATT_BQ;   // first token row of the query tile

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < ATT_KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], SW);
    }
    mbar_init(p_full, SW);
    mbar_init(p_empty, 1);
    mbar_init(o_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, L::TILE);
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c)
        tma_load_3d(smem + L::Q_OFF + c * CHUNK_BYTES, &tmQ, q_full, c * 64, row0, h);
      // K tiles run one ahead of V tiles, in the order in which the tensor pipe frees their stages
      // (QK_{j-1} retires before PV_{j-2}): K_0, K_1, V_0, K_2, V_1, ...
      bool ok = true;
      auto load_k = [&](int j) -> bool {
        const int stage = j % ATT_KV_STAGES;
        if (!mbar_wait(&k_empty[stage], ((uint32_t)(j / ATT_KV_STAGES) & 1) ^ 1, abort_flag, args.status, ST_TIMEOUT_ATTN))
          return false;
        const int kvrow = b * args.S + j * ATT_BKV;
        mbar_expect_tx(&k_full[stage], L::TILE);
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c)
          tma_load_3d(smem + L::K_OFF + stage * L::TILE + c * CHUNK_BYTES, &tmK, &k_full[stage], c * 64, kvrow, hk);
        return true;
      };
      auto load_v = [&](int j) -> bool {
        const int stage = j % ATT_KV_STAGES;
        if (!mbar_wait(&v_empty[stage], ((uint32_t)(j / ATT_KV_STAGES) & 1) ^ 1, abort_flag, args.status, ST_TIMEOUT_ATTN))
          return false;
        const int kvrow = b * args.S + j * ATT_BKV;
        mbar_expect_tx(&v_full[stage], L::TILE);
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c)
          tma_load_3d(smem + L::V_OFF + stage * L::TILE + c * CHUNK_BYTES, &tmV, &v_full[stage], c * 64, kvrow, hk);
        return true;
      };
      ok = load_k(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) ok = load_k(j + 1);
        if (ok) ok = load_v(j);
      }
      if (!ok) {
        // aborting: give copies in flight time to land before the CTA exits
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------------
    // The whole warp runs the loop in lock step and one elected lane issues, so that addresses and descriptors are
    // computed in warp-uniform code (a tcgen05.mma takes them from uniform registers; inside a one-lane branch every
    // operand of every product is first moved there, which cost more than the product itself).  Descriptors are built
    // once; a product adds the 16-byte-unit offset of its contraction step to the address field.
    {
      const bool leader = elect_one();
      const uint32_t tb = __shfl_sync(0xffffffffu, tmem_base, 0);
      constexpr uint32_t idesc_qk = make_idesc_bf16(ATT_BQ, ATT_BKV, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(ATT_BQ, HD, false, true);
      const uint64_t q_desc = make_smem_desc_sw128(smem_u32(smem + L::Q_OFF), 16, 1024);
      const uint64_t k_desc0 = make_smem_desc_sw128(smem_u32(smem + L::K_OFF), 16, 1024);
      const uint64_t v_desc0 = make_smem_desc_sw128(smem_u32(smem + L::V_OFF), CHUNK_BYTES, 1024);
      constexpr uint32_t TILE16 = L::TILE >> 4;
      bool ok = mbar_wait_warp(q_full, 0, abort_flag, args.status, ST_TIMEOUT_ATTN);
      tc_fence_after_sync();
      auto issue_pv = [&](int jj) -> bool {
        const int st = jj % ATT_KV_STAGES;
        const uint32_t kvph = (uint32_t)(jj / ATT_KV_STAGES) & 1;
        if (!mbar_wait_warp(p_full, (uint32_t)jj & 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) return false;
        if (!mbar_wait_warp(&v_full[st], kvph, abort_flag, args.status, ST_TIMEOUT_ATTN)) return false;
        tc_fence_after_sync();
        const uint64_t v_desc = v_desc0 + (uint64_t)(st * TILE16);
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < ATT_BKV / 16; ++kk) {
            // A = P_j straight from tensor memory: 16 keys = 8 columns of packed bf16 pairs per step
            umma_ts(tb + O_COL, tb + P_COL + kk * 8, v_desc + (uint64_t)((kk * 2048) >> 4), idesc_pv,
                    (jj > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&v_empty[st]);    // V_j's stage free again
          umma_commit(p_empty);          // P buffer free, O updated
        }
        return true;
      };
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j % ATT_KV_STAGES;
        const uint32_t kvph = (uint32_t)(j / ATT_KV_STAGES) & 1;
        const int sb = j % S_BUFS;
        const uint32_t sph = (uint32_t)(j / S_BUFS) & 1;
        if (!mbar_wait_warp(&k_full[st], kvph, abort_flag, args.status, ST_TIMEOUT_ATTN) ||
            !mbar_wait_warp(&s_empty[sb], sph ^ 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint64_t k_desc = k_desc0 + (uint64_t)(st * TILE16);
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            const uint64_t o = (uint64_t)(((kk >> 2) * CHUNK_BYTES + (kk & 3) * 32) >> 4);
            umma_ss(tb + sb * 128, q_desc + o, k_desc + o, idesc_qk, kk > 0 ? 1u : 0u);
          }
          umma_commit(&s_full[sb]);
          umma_commit(&k_empty[st]);    // K_j's stage free again as soon as these products retire
        }
        if (j > 0) ok = issue_pv(j - 1);
      }
      if (ok) ok = issue_pv(n_kv - 1);
      if (ok && leader) umma_commit(o_full);
    }
  } else if (SW == 8) {
    // ------------------------------ softmax + epilogue, two warps per 32 rows ----------------
    __shared__ float xmax[2][2][ATT_BQ];       // [tile parity][column half][row]
    __shared__ float xsum[2][ATT_BQ];
    const int quad = warp & 3;                   // tensor-memory lane quarter this warp may touch
    const int half = (warp - 2) >> 2;            // which 64 of the tile's 128 key columns
    const int r = quad * 32 + lane;
    const uint32_t lane_addr = uint32_t(quad * 32) << 16;
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int sb = j % S_BUFS;
      const uint32_t sph = (uint32_t)(j / S_BUFS) & 1;
      if (!mbar_wait(&s_full[sb], sph, abort_flag, args.status, ST_TIMEOUT_ATTN)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t s_addr = tmem_base + sb * 128 + lane_addr + half * 64;
      const bool diag = (j == n_kv - 1);
      // With two CTAs per SM (head_dim 64) a thread has about a hundred registers: the scores are then read twice from
      // tensor memory, 32 columns at a time (once for the maximum, once for the exponentials), instead of being held.
      constexpr bool RELOAD = (HD == 64);
      uint32_t va[32], vb[RELOAD ? 1 : 32];
      auto chunk_max = [&](uint32_t (&v)[32], int col0) -> float {
        if (diag) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if ((col0 + i) > r) v[i] = 0xff800000u;        // -inf: exp2 gives exactly 0
        }
        float m = fmax3(__uint_as_float(v[0]), __uint_as_float(v[1]), __uint_as_float(v[2]));
#pragma unroll
        for (int i = 3; i + 1 < 32; i += 2) m = fmax3(m, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
        return fmaxf(m, __uint_as_float(v[31]));
      };
      float cmax;
      if (RELOAD) {
        tmem_ld_32x32b_x32(s_addr, va);
        tmem_wait_ld();
        cmax = chunk_max(va, half * 64);
        tmem_ld_32x32b_x32(s_addr + 32, va);
        tmem_wait_ld();
        cmax = fmaxf(cmax, chunk_max(va, half * 64 + 32));
      } else {
        uint32_t(&vb2)[32] = *reinterpret_cast<uint32_t(*)[32]>(&vb[0]);
        tmem_ld_32x32b_x32(s_addr, va);
        tmem_ld_32x32b_x32(s_addr + 32, vb2);
        tmem_wait_ld();
        cmax = fmaxf(chunk_max(va, half * 64), chunk_max(vb2, half * 64 + 32));
      }
      // the two warps of a row agree on the tile's maximum (and therefore on every rescaling decision)
      xmax[j & 1][half][r] = cmax;
      pair_barrier(quad);
      const float m_c = fmaxf(cmax, xmax[j & 1][half ^ 1][r]) * args.scale_log2;
      float factor = 1.f;
      bool grow = false;
      if (m_c > m_ref + ATT_RESCALE_THRESHOLD) {
        factor = ex2_approx(m_ref - m_c);       // 0 on the first tile (m_ref = -inf)
        l_sum *= factor;
        m_ref = m_c;
        grow = true;
      }
      uint32_t pk[32];
      float2 lacc2 = make_float2(0.f, 0.f);
      const float2 sc2 = make_float2(args.scale_log2, args.scale_log2);
      const float2 nm2 = make_float2(-m_ref, -m_ref);
      auto chunk_exp = [&](uint32_t (&v)[32], int col0, int out0) {
        if (RELOAD && diag) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if ((col0 + i) > r) v[i] = 0xff800000u;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 t = __ffma2_rn(make_float2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])), sc2, nm2);
          const float2 p2 = make_float2(ex2_approx(t.x), ex2_approx(t.y));
          lacc2 = __fadd2_rn(lacc2, p2);
          pk[out0 + (i >> 1)] = pack_bf16x2(p2.x, p2.y);
        }
      };
      if (RELOAD) {
        tmem_ld_32x32b_x32(s_addr, va);
        tmem_wait_ld();
        chunk_exp(va, half * 64, 0);
        tmem_ld_32x32b_x32(s_addr + 32, va);
        tmem_wait_ld();
        chunk_exp(va, half * 64 + 32, 16);
      } else {
        uint32_t(&vb2)[32] = *reinterpret_cast<uint32_t(*)[32]>(&vb[0]);
        chunk_exp(va, half * 64, 0);
        chunk_exp(vb2, half * 64 + 32, 16);
      }
      l_sum += lacc2.x + lacc2.y;
      // S_j is in registers now: the next QK may overwrite the buffer
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);
      if (j > 0) {
        if (!mbar_wait(p_empty, (uint32_t)(j - 1) & 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (__any_sync(0xffffffffu, grow)) {
          // this warp rescales its half of the output columns
#pragma unroll 1
          for (int c = 0; c < HD / 64; ++c) {
            uint32_t o[32];
            const uint32_t addr = tmem_base + O_COL + lane_addr + half * (HD / 2) + c * 32;
            tmem_ld_32x32b_x32(addr, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
            tmem_st_32x32b_x32(addr, o);
          }
          tmem_wait_st();
        }
      }
      // this warp's 64 keys = 32 packed columns of P
      tmem_st_32x32b_x32(tmem_base + P_COL + lane_addr + half * 32, pk);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- epilogue: O / l -> bf16 (each warp its half of the columns), lse2 ----
    if (ok && mbar_wait(o_full, 0, abort_flag, args.status, ST_TIMEOUT_ATTN)) {
      tc_fence_after_sync();
      xsum[half][r] = l_sum;
      pair_barrier(quad);
      const float l_tot = l_sum + xsum[half ^ 1][r];
      const float inv_l = 1.f / l_tot;
      const long long token = (long long)row0 + r;
      if (ADANA_IN_RANGE(token, (long long)args.B * args.S)) {
        __nv_bfloat16* dst = args.out + token * ((long long)args.Hq * HD) + (long long)h * HD + half * (HD / 2);
#pragma unroll 1
        for (int c = 0; c < HD / 64; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(tmem_base + O_COL + lane_addr + half * (HD / 2) + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 val;
            val.x = pack_bf16x2(__uint_as_float(o[q4 * 8 + 0]) * inv_l, __uint_as_float(o[q4 * 8 + 1]) * inv_l);
            val.y = pack_bf16x2(__uint_as_float(o[q4 * 8 + 2]) * inv_l, __uint_as_float(o[q4 * 8 + 3]) * inv_l);
            val.z = pack_bf16x2(__uint_as_float(o[q4 * 8 + 4]) * inv_l, __uint_as_float(o[q4 * 8 + 5]) * inv_l);
            val.w = pack_bf16x2(__uint_as_float(o[q4 * 8 + 6]) * inv_l, __uint_as_float(o[q4 * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = val;
          }
        }
        if (half == 0) args.lse2[((long long)b * args.Hq + h) * args.S + qt * ATT_BQ + r] = m_ref + log2f(l_tot);
      }
    }
  } else {
    // ------------------------------ softmax + epilogue (warps 2..5) -------------------------
    const int quad = warp & 3;
    const int r = quad * 32 + lane;              // query row inside the tile
    const uint32_t lane_addr = uint32_t(quad * 32) << 16;
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int sb = j % S_BUFS;
      const uint32_t sph = (uint32_t)(j / S_BUFS) & 1;
      if (!mbar_wait(&s_full[sb], sph, abort_flag, args.status, ST_TIMEOUT_ATTN)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t s_addr = tmem_base + sb * 128 + lane_addr;
      const bool diag = (j == n_kv - 1);
      // One pass over the row, 32 columns at a time; the next chunk's tensor-memory load is in
      // flight while the current one is processed.  Probabilities are taken relative to the running
      // reference maximum m_ref, which only moves when a chunk exceeds it by more than 2^8; then
      // the row sum, the chunks already packed and (later) the output accumulator are rescaled.
      // Only the diagonal tile pays for masking.  The arithmetic is packed two columns per
      // instruction (f32x2 FMA / add, three-input max) because this loop, not the tensor pipe,
      // bounds the kernel at head_dim 64.
      uint32_t pk[64];
      float2 lacc2 = make_float2(0.f, 0.f);
      float o_factor = 1.f;
      uint32_t va[32], vb[32];
      tmem_ld_32x32b_x32(s_addr, va);
      tmem_wait_ld();
      const float2 sc2 = make_float2(args.scale_log2, args.scale_log2);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t(&cur)[32] = (c & 1) ? vb : va;
        uint32_t(&nxt)[32] = (c & 1) ? va : vb;
        if (c < 3) tmem_ld_32x32b_x32(s_addr + (c + 1) * 32, nxt);
        if (diag) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if ((c * 32 + i) > r) cur[i] = 0xff800000u;  // -inf: exp2 gives exactly 0
        }
        float cmax = fmax3(__uint_as_float(cur[0]), __uint_as_float(cur[1]), __uint_as_float(cur[2]));
#pragma unroll
        for (int i = 3; i + 1 < 32; i += 2)
          cmax = fmax3(cmax, __uint_as_float(cur[i]), __uint_as_float(cur[i + 1]));
        cmax = fmaxf(cmax, __uint_as_float(cur[31]));
        const float m_c = cmax * args.scale_log2;
        if (m_c > m_ref + ATT_RESCALE_THRESHOLD) {
          const float f = ex2_approx(m_ref - m_c);      // 0 on the very first chunk (m_ref = -inf)
          l_sum *= f;
          lacc2.x *= f;
          lacc2.y *= f;
          o_factor *= f;
#pragma unroll
          for (int cc = 0; cc < c; ++cc) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float2 pv = unpack_bf16x2(pk[cc * 16 + i]);
              pk[cc * 16 + i] = pack_bf16x2(pv.x * f, pv.y * f);
            }
          }
          m_ref = m_c;
        }
        const float2 nm2 = make_float2(-m_ref, -m_ref);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 t = __ffma2_rn(make_float2(__uint_as_float(cur[i]), __uint_as_float(cur[i + 1])), sc2, nm2);
          const float2 p2 = make_float2(ex2_approx(t.x), ex2_approx(t.y));
          lacc2 = __fadd2_rn(lacc2, p2);
          pk[c * 16 + (i >> 1)] = pack_bf16x2(p2.x, p2.y);
        }
        if (c < 3) tmem_wait_ld();
      }
      const float lacc = lacc2.x + lacc2.y;
      l_sum += lacc;
      const bool grow = o_factor != 1.f;
      const float factor = o_factor;
      // S_j is in registers now: the next QK may overwrite the buffer
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);
      // P buffer / O accumulator are free once PV_{j-1} retired
      if (j > 0) {
        if (!mbar_wait(p_empty, (uint32_t)(j - 1) & 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (__any_sync(0xffffffffu, grow)) {
          // rescale the running output (tensor memory) by exp2(m_old - m_new); lanes that did not
          // grow multiply by one
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(tmem_base + O_COL + lane_addr + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
            tmem_st_32x32b_x32(tmem_base + O_COL + lane_addr + c * 32, o);
          }
          tmem_wait_st();
        }
      }
      // P_j (bf16 pairs) goes to tensor memory, where the PV MMA reads it as its A operand: lane r
      // writes its row's 64 packed columns
      {
        uint32_t(&lo)[32] = *reinterpret_cast<uint32_t(*)[32]>(&pk[0]);
        uint32_t(&hi)[32] = *reinterpret_cast<uint32_t(*)[32]>(&pk[32]);
        tmem_st_32x32b_x32(tmem_base + P_COL + lane_addr, lo);
        tmem_st_32x32b_x32(tmem_base + P_COL + lane_addr + 32, hi);
        tmem_wait_st();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- epilogue: O / l -> bf16, lse2 ----
    if (ok && mbar_wait(o_full, 0, abort_flag, args.status, ST_TIMEOUT_ATTN)) {
      tc_fence_after_sync();
      const float inv_l = 1.f / l_sum;
      const long long token = (long long)row0 + r;
      if (ADANA_IN_RANGE(token, (long long)args.B * args.S)) {
      __nv_bfloat16* dst = args.out + token * ((long long)args.Hq * HD) + (long long)h * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(tmem_base + O_COL + lane_addr + c * 32, o);
        tmem_wait_ld();
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 val;
          val.x = pack_bf16x2(__uint_as_float(o[q4 * 8 + 0]) * inv_l, __uint_as_float(o[q4 * 8 + 1]) * inv_l);
          val.y = pack_bf16x2(__uint_as_float(o[q4 * 8 + 2]) * inv_l, __uint_as_float(o[q4 * 8 + 3]) * inv_l);
          val.z = pack_bf16x2(__uint_as_float(o[q4 * 8 + 4]) * inv_l, __uint_as_float(o[q4 * 8 + 5]) * inv_l);
          val.w = pack_bf16x2(__uint_as_float(o[q4 * 8 + 6]) * inv_l, __uint_as_float(o[q4 * 8 + 7]) * inv_l);
          *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = val;
        }
      }
      args.lse2[((long long)b * args.Hq + h) * args.S + qt * ATT_BQ + r] = m_ref + log2f(l_sum);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int HD, int S_BUFS, int SW>
static int launch_attn_fwd_sw(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                              const AttFwdArgs& a, cudaStream_t st) {
  auto kern = attn_fwd_kernel<HD, S_BUFS, SW>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, AttFwdSmem<HD>::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int grid = a.B * a.Hq * (a.S / ATT_BQ);
  kern<<<grid, 64 + 32 * SW, AttFwdSmem<HD>::TOTAL, st>>>(tq, tk, tv, a);
  return (int)cudaGetLastError();
}

// ---- forward, two softmax groups on alternate key tiles ------------------------------------------------------------
// A clock trace of the kernel above showed its softmax warps as the critical path, and only half of their time per
// tile in the exponentials: the rest (tensor-memory loads, row maximum, hand-offs) left the exponential unit idle,
// because all softmax warps of the CTA go through the same phase at the same time.  Here one CTA per SM runs TWO groups
// of four softmax warps: group g takes the key tiles j = g (mod 2) and keeps its own running reference maximum, row sum
// and output accumulator O_g, so the groups never wait for one another and one group's exponentials run under the other
// group's loads and hand-offs.  A group is eight warps, two per 32 rows, each taking 64 of the tile's 128 key columns
// (the pair agrees on the row maximum through shared memory, as above): sixteen softmax warps per SM, four per
// scheduler, which is what it takes to keep the exponential unit fed while other warps are between phases.
// Tensor memory: S_0 | S_1 | O_0 | O_1; P_j is written over the first 64 columns of its
// own S_j (free once the scores are in registers).  The tensor pipe runs QK_0, QK_1, PV_0, QK_2, PV_1, ...; products of
// one thread retire in order, so QK_{j+2} cannot overwrite S_j / P_j before PV_j has read it, and "S_{j+2} is full"
// implies "PV_j has retired", which is all a group needs before it rescales O_g.  The epilogue joins the two streams:
// out = (2^(m_0 - m) O_0 + 2^(m_1 - m) O_1) / (2^(m_0 - m) l_0 + 2^(m_1 - m) l_1), m = max(m_0, m_1).
template <int HD>
struct AttFwdPPSmem {
  static constexpr int STAGES = HD == 64 ? 4 : 2;
  static constexpr int TILE = ATT_BQ * HD * 2;
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = TILE;
  static constexpr int V_OFF = K_OFF + STAGES * TILE;
  static constexpr int BAR_OFF = V_OFF + STAGES * TILE;
  static constexpr int TOTAL = BAR_OFF + 512;
};
constexpr int ATT_PP_THREADS = 576;       // TMA warp, MMA warp, 2 groups x 8 softmax warps

template <int HD>
__global__ void __launch_bounds__(ATT_PP_THREADS, 1)
attn_fwd_pp_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const AttFwdArgs args) {
  using L = AttFwdPPSmem<HD>;
  constexpr int STAGES = L::STAGES;
  constexpr int CHUNKS = HD / 64;
  constexpr int CHUNK_BYTES = ATT_BQ * 128;
  constexpr uint32_t O_COL = 256;                  // O_g at O_COL + g * HD
  constexpr uint32_t TMEM_COLS = 512;

  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* q_full = bars;                 // [1]
  uint64_t* k_full = bars + 1;             // [STAGES]
  uint64_t* v_full = bars + 1 + STAGES;    // [STAGES]
  uint64_t* k_empty = bars + 1 + 2 * STAGES;
  uint64_t* v_empty = bars + 1 + 3 * STAGES;
  uint64_t* s_full = bars + 1 + 4 * STAGES;      // [2]
  uint64_t* p_full = s_full + 2;                 // [2]
  uint64_t* o_full = p_full + 2;                 // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  __shared__ float xm[2][ATT_BQ], xl[2][2][ATT_BQ];      // [group][row], [group][column half][row]
  __shared__ float xmax[2][2][2][ATT_BQ];                // [group][tile parity][column half][row]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = args.S / ATT_BQ;
  const int BH = args.B * args.Hq;
  const int qt = n_qt - 1 - (int)(blockIdx.x / BH);      // heaviest query tiles first
  const int bh = (int)(blockIdx.x % BH);
  const int b = bh / args.Hq, h = bh % args.Hq;
  const int hk = h / (args.Hq / args.Hk);
  const int n_kv = qt + 1;
  const int row0 = b * args.S + qt * ATT_BQ;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(&s_full[g], 1);
      mbar_init(&p_full[g], 8);
    }
    mbar_init(o_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, L::TILE);
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c)
        tma_load_3d(smem + L::Q_OFF + c * CHUNK_BYTES, &tmQ, q_full, c * 64, row0, h);
      bool ok = true;
      auto load_k = [&](int j) -> bool {
        const int stage = j % STAGES;
        if (!mbar_wait(&k_empty[stage], ((uint32_t)(j / STAGES) & 1) ^ 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) return false;
        const int kvrow = b * args.S + j * ATT_BKV;
        mbar_expect_tx(&k_full[stage], L::TILE);
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c)
          tma_load_3d(smem + L::K_OFF + stage * L::TILE + c * CHUNK_BYTES, &tmK, &k_full[stage], c * 64, kvrow, hk);
        return true;
      };
      auto load_v = [&](int j) -> bool {
        const int stage = j % STAGES;
        if (!mbar_wait(&v_empty[stage], ((uint32_t)(j / STAGES) & 1) ^ 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) return false;
        const int kvrow = b * args.S + j * ATT_BKV;
        mbar_expect_tx(&v_full[stage], L::TILE);
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c)
          tma_load_3d(smem + L::V_OFF + stage * L::TILE + c * CHUNK_BYTES, &tmV, &v_full[stage], c * 64, kvrow, hk);
        return true;
      };
      // K tiles run two ahead of V tiles, following the order in which the tensor pipe frees their stages
      ok = load_k(0);
      if (ok && n_kv > 1) ok = load_k(1);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 2 < n_kv) ok = load_k(j + 2);
        if (ok) ok = load_v(j);
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();      // aborting: give copies in flight time to land before the CTA exits
        while (globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (warp-uniform loop, one elected lane issues) --------------
    const bool leader = elect_one();
    const uint32_t tb = __shfl_sync(0xffffffffu, tmem_base, 0);
    constexpr uint32_t idesc_qk = make_idesc_bf16(ATT_BQ, ATT_BKV, false, false);
    constexpr uint32_t idesc_pv = make_idesc_bf16(ATT_BQ, HD, false, true);
    const uint64_t q_desc = make_smem_desc_sw128(smem_u32(smem + L::Q_OFF), 16, 1024);
    const uint64_t k_desc0 = make_smem_desc_sw128(smem_u32(smem + L::K_OFF), 16, 1024);
    const uint64_t v_desc0 = make_smem_desc_sw128(smem_u32(smem + L::V_OFF), CHUNK_BYTES, 1024);
    constexpr uint32_t TILE16 = L::TILE >> 4;
    bool ok = mbar_wait_warp(q_full, 0, abort_flag, args.status, ST_TIMEOUT_ATTN);
    tc_fence_after_sync();
    auto issue_qk = [&](int j) -> bool {
      const int st = j % STAGES;
      if (!mbar_wait_warp(&k_full[st], (uint32_t)(j / STAGES) & 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) return false;
      tc_fence_after_sync();
      const uint64_t k_desc = k_desc0 + (uint64_t)(st * TILE16);
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint64_t o = (uint64_t)(((kk >> 2) * CHUNK_BYTES + (kk & 3) * 32) >> 4);
          umma_ss(tb + (j & 1) * 128, q_desc + o, k_desc + o, idesc_qk, kk > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[j & 1]);
        umma_commit(&k_empty[st]);
      }
      return true;
    };
    auto issue_pv = [&](int j) -> bool {
      const int st = j % STAGES, g = j & 1;
      if (!mbar_wait_warp(&p_full[g], (uint32_t)(j >> 1) & 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) return false;
      if (!mbar_wait_warp(&v_full[st], (uint32_t)(j / STAGES) & 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) return false;
      tc_fence_after_sync();
      const uint64_t v_desc = v_desc0 + (uint64_t)(st * TILE16);
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < ATT_BKV / 16; ++kk)
          umma_ts(tb + O_COL + g * HD, tb + g * 128 + kk * 8, v_desc + (uint64_t)((kk * 2048) >> 4), idesc_pv,
                  (j > 1 || kk > 0) ? 1u : 0u);
        umma_commit(&v_empty[st]);
      }
      return true;
    };
    if (ok) ok = issue_qk(0);
    for (int j = 1; j < n_kv && ok; ++j) {
      ok = issue_qk(j);                  // S_{j&1} / P_{j-2}: the products of this thread retire in order, so PV_{j-2} has read
      if (ok) ok = issue_pv(j - 1);      // its P before these scores land
    }
    if (ok) ok = issue_pv(n_kv - 1);
    if (ok && leader) umma_commit(o_full);
  } else {
    // ------------------------------ softmax groups: warps 2..9 even tiles, warps 10..17 odd tiles -------------
    const int g = (warp - 2) >> 3;
    const int half = ((warp - 2) >> 2) & 1;          // which 64 of the tile's 128 key columns
    const int quad = warp & 3;                        // tensor-memory lane quarter this warp may touch
    const int r = quad * 32 + lane;
    const uint32_t lane_addr = uint32_t(quad * 32) << 16;
    const uint32_t s_addr = tmem_base + g * 128 + lane_addr + half * 64;
    const uint32_t o_addr = tmem_base + O_COL + g * HD + lane_addr + half * (HD / 2);
    const int pair_id = 1 + g * 4 + quad;
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = g; j < n_kv && ok; j += 2) {
      if (!mbar_wait(&s_full[g], (uint32_t)(j >> 1) & 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const bool diag = (j == n_kv - 1);
      const int par = (j >> 1) & 1;
      // about a hundred registers per thread: the scores are read twice from tensor memory, 32 columns at a time
      // (once for the maximum, once for the exponentials), instead of being held
      uint32_t va[32];
      auto chunk_mask = [&](int col0) {
        if (diag) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if ((col0 + i) > r) va[i] = 0xff800000u;        // -inf: exp2 gives exactly 0
        }
      };
      auto chunk_max = [&]() -> float {
        float m = fmax3(__uint_as_float(va[0]), __uint_as_float(va[1]), __uint_as_float(va[2]));
#pragma unroll
        for (int i = 3; i + 1 < 32; i += 2) m = fmax3(m, __uint_as_float(va[i]), __uint_as_float(va[i + 1]));
        return fmaxf(m, __uint_as_float(va[31]));
      };
      tmem_ld_32x32b_x32(s_addr, va);
      tmem_wait_ld();
      chunk_mask(half * 64);
      float cmax = chunk_max();
      tmem_ld_32x32b_x32(s_addr + 32, va);
      tmem_wait_ld();
      chunk_mask(half * 64 + 32);
      cmax = fmaxf(cmax, chunk_max());
      // the two warps of a row agree on the tile's maximum (and therefore on every rescaling decision)
      xmax[g][par][half][r] = cmax;
      named_barrier_sync(pair_id, 64);
      const float m_c = fmaxf(cmax, xmax[g][par][half ^ 1][r]) * args.scale_log2;
      float factor = 1.f;
      bool grow = false;
      if (m_c > m_ref + ATT_RESCALE_THRESHOLD) {
        factor = ex2_approx(m_ref - m_c);       // 0 on the group's first tile (m_ref = -inf)
        l_sum *= factor;
        m_ref = m_c;
        grow = true;
      }
      uint32_t pk[32];
      float2 lacc2 = make_float2(0.f, 0.f);
      const float2 sc2 = make_float2(args.scale_log2, args.scale_log2);
      const float2 nm2 = make_float2(-m_ref, -m_ref);
      auto chunk_exp = [&](int out0) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 t = __ffma2_rn(make_float2(__uint_as_float(va[i]), __uint_as_float(va[i + 1])), sc2, nm2);
          const float2 p2 = make_float2(ex2_approx(t.x), ex2_approx(t.y));
          lacc2 = __fadd2_rn(lacc2, p2);
          pk[out0 + (i >> 1)] = pack_bf16x2(p2.x, p2.y);
        }
      };
      chunk_exp(16);                             // the second 32 columns are still in registers
      tmem_ld_32x32b_x32(s_addr, va);
      tmem_wait_ld();
      // (the warp with keys 0..63 has now read all its scores: its partner may overwrite columns 32..63 with P)
      if (half == 0) {
        tc_fence_before_sync();
        named_barrier_arrive(pair_id, 64);
      }
      chunk_mask(half * 64);
      chunk_exp(0);
      l_sum += lacc2.x + lacc2.y;
      if (j >= 2 && __any_sync(0xffffffffu, grow)) {
        // PV_{j-2} has retired (it precedes QK_j in the tensor pipe): rescale this warp's half of the group's accumulator
#pragma unroll 1
        for (int c = 0; c < HD / 64; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(o_addr + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
          tmem_st_32x32b_x32(o_addr + c * 32, o);
        }
        tmem_wait_st();
      }
      // P_j over the first 64 columns of S_j: this warp's 64 keys are 32 packed columns.  The warp with keys 64..127
      // writes columns 32..63, which hold scores of its partner: it waits until the partner has read them
      if (half == 1) {
        named_barrier_sync(pair_id, 64);
        tc_fence_after_sync();
      }
      tmem_st_32x32b_x32(tmem_base + g * 128 + lane_addr + half * 32, pk);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[g]);
    }
    // ---- epilogue: join the two streams; every (group, half) writes a quarter of the output columns ----
    if (half == 0) xm[g][r] = m_ref;
    xl[g][half][r] = l_sum;
    named_barrier_sync(9, 512);
    if (ok && mbar_wait(o_full, 0, abort_flag, args.status, ST_TIMEOUT_ATTN)) {
      tc_fence_after_sync();
      const bool two = n_kv > 1;                       // with one key tile the odd group never ran: O_1 holds nothing
      const float m0 = xm[0][r], m1 = two ? xm[1][r] : -INFINITY;
      const float m = fmaxf(m0, m1);
      const float w0 = ex2_approx(m0 - m), w1 = two ? ex2_approx(m1 - m) : 0.f;
      const float l_tot = (xl[0][0][r] + xl[0][1][r]) * w0 + (two ? (xl[1][0][r] + xl[1][1][r]) * w1 : 0.f);
      const float inv_l = 1.f / l_tot;
      const float a0 = w0 * inv_l, a1 = w1 * inv_l;
      const long long token = (long long)row0 + r;
      constexpr int QC = HD / 4;                       // output columns of this warp
      const int c0 = (g * 2 + half) * QC;
      if (ADANA_IN_RANGE(token, (long long)args.B * args.S)) {
        __nv_bfloat16* dst = args.out + token * ((long long)args.Hq * HD) + (long long)h * HD + c0;
        const uint32_t oa = tmem_base + O_COL + lane_addr + c0;
#pragma unroll 1
        for (int c = 0; c < QC / 16; ++c) {
          uint32_t o0[16], o1[16];
          tmem_ld_32x32b_x16(oa + c * 16, o0);
          if (two) tmem_ld_32x32b_x16(oa + HD + c * 16, o1);
          tmem_wait_ld();
#pragma unroll
          for (int q4 = 0; q4 < 2; ++q4) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e)
              f[e] = __uint_as_float(o0[q4 * 8 + e]) * a0 + (two ? __uint_as_float(o1[q4 * 8 + e]) * a1 : 0.f);
            uint4 val;
            val.x = pack_bf16x2(f[0], f[1]);
            val.y = pack_bf16x2(f[2], f[3]);
            val.z = pack_bf16x2(f[4], f[5]);
            val.w = pack_bf16x2(f[6], f[7]);
            *reinterpret_cast<uint4*>(dst + c * 16 + q4 * 8) = val;
          }
        }
        if (g == 0 && half == 0) args.lse2[((long long)b * args.Hq + h) * args.S + qt * ATT_BQ + r] = m + log2f(l_tot);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int HD>
static int launch_attn_fwd_pp(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttFwdArgs& a,
                              cudaStream_t st) {
  auto kern = attn_fwd_pp_kernel<HD>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, AttFwdPPSmem<HD>::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int grid = a.B * a.Hq * (a.S / ATT_BQ);
  kern<<<grid, ATT_PP_THREADS, AttFwdPPSmem<HD>::TOTAL, st>>>(tq, tk, tv, a);
  return (int)cudaGetLastError();
}

template <int HD, int S_BUFS>
static int launch_attn_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                           const AttFwdArgs& a, cudaStream_t st) {
  // Default: the single-stream kernel at the top of this file, with four softmax warps and two CTAs per SM at head_dim
  // 64 and eight softmax warps at head_dim 128 (ADANA_ATT_FWD_SW overrides).  ADANA_ATT_FWD=pp selects the kernel with
  // two softmax groups on alternate key tiles: its steady state is faster (1758 against 2179 clocks per key tile at
  // head_dim 128), but with one CTA per SM nothing hides the start and the epilogue of a CTA, and over whole problems
  // it measures 3 % behind at head_dim 128 and 20 % behind at head_dim 64; it needs a persistent tile loop to pay off.
  static int sw = -1;
  if (sw < 0) {
    const char* f = getenv("ADANA_ATT_FWD");
    const char* e = getenv("ADANA_ATT_FWD_SW");
    if (f && f[0] == 'p') sw = 0;
    else sw = (e && atoi(e) == 8) ? 8 : (e && atoi(e) == 4) ? 4 : (HD == 128 ? 8 : 4);
  }
  if (sw == 0) return launch_attn_fwd_pp<HD>(tq, tk, tv, a, st);
  return sw == 4 ? launch_attn_fwd_sw<HD, S_BUFS, 4>(tq, tk, tv, a, st) : launch_attn_fwd_sw<HD, S_BUFS, 8>(tq, tk, tv, a, st);
}

}  // namespace adana

using namespace adana;

// q [T, Hq, hd], k [T, Hk, hd] contiguous bf16; v read from `vbase` with row pitch `ldv` and head
// pitch `v_hstride` (elements); out [T, Hq*hd] bf16; lse2 [B, Hq, S] fp32.
extern "C" int adana_attn_fwd(const void* q, const void* k, const void* vbase, long long ldv,
                              int v_hstride, void* out, float* lse2, int B, int S, int Hq, int Hk,
                              int hd, float scale, int* status, void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (B <= 0 || S <= 0) return 0;
  if ((hd != 64 && hd != 128) || (S % ATT_BQ) != 0 || Hq % Hk != 0) return -1;
  const uint64_t T = (uint64_t)B * S;
  CUtensorMap tq, tk, tv;
  {
    uint64_t dims[3] = {(uint64_t)hd, T, (uint64_t)Hq};
    uint64_t str[3] = {1, (uint64_t)Hq * hd, (uint64_t)hd};
    uint32_t box[3] = {64, ATT_BQ, 1};
    if (encode_tmap_nd(&tq, q, 3, dims, str, box, 2, 1)) return -2;
  }
  {
    uint64_t dims[3] = {(uint64_t)hd, T, (uint64_t)Hk};
    uint64_t str[3] = {1, (uint64_t)Hk * hd, (uint64_t)hd};
    uint32_t box[3] = {64, ATT_BKV, 1};
    if (encode_tmap_nd(&tk, k, 3, dims, str, box, 2, 1)) return -3;
  }
  {
    uint64_t dims[3] = {(uint64_t)hd, T, (uint64_t)Hk};
    uint64_t str[3] = {1, (uint64_t)ldv, (uint64_t)v_hstride};
    uint32_t box[3] = {64, ATT_BKV, 1};
    if (encode_tmap_nd(&tv, vbase, 3, dims, str, box, 2, 1)) return -4;
  }
  AttFwdArgs a;
  a.out = (__nv_bfloat16*)out;
  a.lse2 = lse2;
  a.B = B; a.S = S; a.Hq = Hq; a.Hk = Hk;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  if (hd == 64) return launch_attn_fwd<64, 1>(tq, tk, tv, a, st);
  return launch_attn_fwd<128, 2>(tq, tk, tv, a, st);
}

namespace adana {

// =================================================================================================
// Backward.
//
// One CTA = one (batch, KV head, 128-key tile j); K_j and V_j stay in shared memory while the CTA
// walks every (query head of the group, query tile i >= j).  The scores are computed TRANSPOSED, so
// that a tensor-memory lane is a key row and the probabilities can feed the dV / dK products
// straight from tensor memory (operand A of a tcgen05.mma may live there; a lane is a row of A):
//     S^T  = K_j Q_i^T          dP^T = V_j dO_i^T                     (tensor memory, fp32)
//     P^T  = exp2(scale*S^T - lse2[q])        -> bf16, written over S^T in tensor memory
//     dS^T = P^T o (dP^T - delta[q]) * scale  -> bf16, written over dP^T in tensor memory AND to shared memory
//     dV_j += P^T dO_i          dK_j += dS^T Q_i                      (A from tensor memory)
//     dQ_i  = dS K_j            (A = the shared-memory dS^T tile read M-major) -> TMA reduce-adds into fp32 dQ
// Shared-memory bandwidth, not the tensor pipe, bounds this kernel (an M=128, N=64 product with both operands
// in shared memory moves 6 KB per 32 tensor cycles), so P never touches shared memory and dV / dK read only
// their B operand from it.
//
// Roles: warp 0 TMA producer (Q_i, dO_i and the tile's 128 lse2 / delta values per item), warp 1 MMA issuer,
// warps 2..9 exponential warps (S^T -> P^T; warp w owns the tensor-memory lane quarter w % 4 = 32 key rows, the
// two warps of a quarter split the 128 query columns), warps 10..13 dS warps (P^T, dP^T -> dS^T for a whole key
// row per thread, then the drain of the previous item's dQ).  The exponentials are bound by the special-function
// unit and need two warps per scheduler to keep it busy; the dS arithmetic is bound by the FMA pipe and by
// instruction issue: in separate warps the two overlap, and the single S^T region only has to wait for the
// exponentials, not for the dS pass.
//
// Tensor-memory columns (512):   head_dim 64: S^T | dP^T x2 | dV | dK      head_dim 128: S^T | dP^T | dV | dK
// Packed bf16 P^T takes columns [0,32) and [64,96) of the S^T region (each column half overwrites only fp32
// columns it has already loaded); packed dS^T takes columns [0,64) of its dP^T region.  dQ_i lands in columns
// [64,128) of its item's dP^T region (head_dim 64) or over the S^T region (head_dim 128, where P^T has been
// consumed by then).
// head_dim 64: with two dP^T regions and two dS^T tiles the chain of an item (dP^T -> dS^T -> dK, dQ -> drain)
// overlaps the next item's (S^T -> P^T -> dV); head_dim 128 has no columns to spare and runs the items back
// to back.  lse2 and `delta` are per QUERY, i.e. per column here: every lane reads the same staged values.
// =================================================================================================
template <int HD>
struct AttBwdSmem {
  static constexpr int TILE = ATT_BQ * HD * 2;
  static constexpr int STAGES = (HD == 64) ? 3 : 1;        // Q / dO ring: a TMA load takes longer than an item
  static constexpr int DS_BUFS = (HD == 64) ? 2 : 1;
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = TILE;
  static constexpr int Q_OFF = 2 * TILE;
  static constexpr int DO_OFF = Q_OFF + STAGES * TILE;
  static constexpr int DS_OFF = DO_OFF + STAGES * TILE;                    // dS^T tiles [128 keys][128 queries] bf16
  static constexpr int DQ_OFF = DS_OFF + DS_BUFS * ATT_BQ * ATT_BKV * 2;   // fp32 dQ staging: 4 warps x 1 box [32][32]
  static constexpr int DQ_BOX = 32 * 128;
  static constexpr int STAT_OFF = DQ_OFF + 4 * DQ_BOX;                     // per stage: lse2[128] | ndelta[128]
  static constexpr int BAR_OFF = STAT_OFF + STAGES * 1024;
  static constexpr int TOTAL = BAR_OFF + 256;
};

struct AttBwdArgs {
  const float* lse2;      // [B, Hq, S]
  const float* ndelta;    // [B, Hq, S]: -scale * rowsum(dO o O)
  float* dq_acc;          // [T, Hq, HD] fp32, cleared by the delta kernel that runs before this one
  __nv_bfloat16* dk;      // [T, Hk, HD]
  __nv_bfloat16* dv;      // base of the v columns in the projection-gradient buffer
  long long lddv;
  int dv_hstride;
  int B, S, Hq, Hk;
  float scale, scale_log2;
  int* status;
};

template <int HD>
__global__ void __launch_bounds__(ATT_BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                const __grid_constant__ CUtensorMap tmDQ, const AttBwdArgs args) {
  using L = AttBwdSmem<HD>;
  constexpr int CHUNKS = HD / 64;
  constexpr int CHUNK_BYTES = ATT_BQ * 128;
  constexpr int STAGES = L::STAGES;
  constexpr int DPT_BUFS = (HD == 64) ? 2 : 1;
  constexpr bool OVERLAP = (HD == 64);
  constexpr uint32_t ST_COL = 0, DPT_COL = 128, DV_COL = DPT_COL + DPT_BUFS * 128, DK_COL = DV_COL + HD;
  constexpr uint32_t DQ_IN_DPT = 64;      // head_dim 64: dQ's columns inside its item's dP^T region
  static_assert(DK_COL + HD == 512, "tensor-memory plan must fill 512 columns");
  static_assert(L::TOTAL <= 227 * 1024, "shared memory plan");

  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* kv_full = bars;            // [1]
  uint64_t* qdo_full = bars + 1;       // [4]
  uint64_t* qdo_empty = bars + 5;      // [4]
  uint64_t* st_full = bars + 9;        // [1]  MMA: S^T of an item is in tensor memory
  uint64_t* p_full = bars + 10;        // [2]  score warps: P^T written                       (by item parity)
  uint64_t* dpt_full = bars + 12;      // [2]  MMA: dP^T is in tensor memory                  (by item parity)
  uint64_t* ds_full = bars + 14;       // [2]  score warps: dS^T in tensor and shared memory  (by item parity)
  uint64_t* dq_full = bars + 16;       // [2]  MMA: dK / dQ products of the item retired      (by item parity)
  uint64_t* dq_free = bars + 18;       // [2]  drain warps: dQ drained                        (by item parity)
  uint64_t* acc_full = bars + 20;
  uint64_t* p_read = bars + 21;        // [2]  dS warps: P^T is in their registers (S^T may be overwritten)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 23);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_t = args.S / ATT_BQ;
  const int G = args.Hq / args.Hk;
  const int BHk = args.B * args.Hk;
  // KV tile 0 has the most query tiles: schedule it first
  const int j = (int)(blockIdx.x / BHk);
  const int bhk = (int)(blockIdx.x % BHk);
  const int b = bhk / args.Hk, hk = bhk % args.Hk;
  const int n_i = n_t - j;                 // query tiles i = j .. n_t-1
  const int n_items = G * n_i;
  const int kvrow = b * args.S + j * ATT_BKV;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(st_full, 1);
    for (int s = 0; s < 4; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&p_full[s], 8);
      mbar_init(&p_read[s], 4);
      mbar_init(&dpt_full[s], 1);
      mbar_init(&ds_full[s], 4);
      mbar_init(&dq_full[s], 1);
      mbar_init(&dq_free[s], 4);
    }
    mbar_init(acc_full, 1);
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
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmDO);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(kv_full, 2 * L::TILE);
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        tma_load_3d(smem + L::K_OFF + c * CHUNK_BYTES, &tmK, kv_full, c * 64, kvrow, hk);
        tma_load_3d(smem + L::V_OFF + c * CHUNK_BYTES, &tmV, kv_full, c * 64, kvrow, hk);
      }
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = 0; t < n_items && ok; ++t) {
        const int g = t / n_i, i = j + t % n_i;
        const int hq = hk * G + g;
        const int qrow = b * args.S + i * ATT_BQ;
        if (!mbar_wait(&qdo_empty[stage], phase ^ 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) {
          ok = false;
          break;
        }
        mbar_expect_tx(&qdo_full[stage], 2 * L::TILE + 1024);
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
          tma_load_3d(smem + L::Q_OFF + stage * L::TILE + c * CHUNK_BYTES, &tmQ, &qdo_full[stage], c * 64, qrow, hq);
          tma_load_3d(smem + L::DO_OFF + stage * L::TILE + c * CHUNK_BYTES, &tmDO, &qdo_full[stage], c * 64, qrow, hq);
        }
        const long long stat = ((long long)b * args.Hq + hq) * args.S + i * ATT_BQ;
        bulk_load_1d(smem + L::STAT_OFF + stage * 1024, args.lse2 + stat, 512, &qdo_full[stage]);
        bulk_load_1d(smem + L::STAT_OFF + stage * 1024 + 512, args.ndelta + stat, 512, &qdo_full[stage]);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------------
    // The whole warp runs this loop in lock step and one elected lane issues: addresses and descriptors are then
    // computed in warp-uniform code instead of inside a divergent branch.
    {
      const bool leader = elect_one();
      const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);
      constexpr uint32_t idesc_s = make_idesc_bf16(ATT_BKV, ATT_BQ, false, false);   // K Q^T, V dO^T (both K-major)
      constexpr uint32_t idesc_ts = make_idesc_bf16(ATT_BKV, HD, false, true);       // P^T dO, dS^T Q (A in tensor memory)
      constexpr uint32_t idesc_dq = make_idesc_bf16(ATT_BQ, HD, true, true);         // dS K (A = dS^T tile read M-major)
      // One thread issues every product, so its instruction count per product matters: the shared-memory descriptors
      // are built once, and a product only adds the 16-byte-unit offset of its contraction step to the address field
      // (the low 14 bits; tiles sit below 256 KB, so the sum never carries out of it).
      const uint64_t k_kmaj = make_smem_desc_sw128(smem_u32(smem + L::K_OFF), 16, 1024);
      const uint64_t v_kmaj = make_smem_desc_sw128(smem_u32(smem + L::V_OFF), 16, 1024);
      const uint64_t k_mnmaj = make_smem_desc_sw128(smem_u32(smem + L::K_OFF), CHUNK_BYTES, 1024);
      const uint64_t q_kmaj0 = make_smem_desc_sw128(smem_u32(smem + L::Q_OFF), 16, 1024);
      const uint64_t q_mnmaj0 = make_smem_desc_sw128(smem_u32(smem + L::Q_OFF), CHUNK_BYTES, 1024);
      const uint64_t do_kmaj0 = make_smem_desc_sw128(smem_u32(smem + L::DO_OFF), 16, 1024);
      const uint64_t do_mnmaj0 = make_smem_desc_sw128(smem_u32(smem + L::DO_OFF), CHUNK_BYTES, 1024);
      const uint64_t ds_mnmaj0 = make_smem_desc_sw128(smem_u32(smem + L::DS_OFF), CHUNK_BYTES, 1024);
      constexpr uint32_t TILE16 = L::TILE >> 4, DS16 = (ATT_BQ * ATT_BKV * 2) >> 4;
      // 16-byte units: K-major step kk of a tile (64-column chunks CHUNK_BYTES apart), MN-major step kk (16 rows)
#define KMAJ_STEP(kk) (uint64_t)((((kk) >> 2) * CHUNK_BYTES + ((kk) & 3) * 32) >> 4)
#define MNMAJ_STEP(kk) (uint64_t)(((kk) * 2048) >> 4)
      bool ok = mbar_wait_warp(kv_full, 0, abort_flag, args.status, ST_TIMEOUT_ATTN);
      tc_fence_after_sync();

      auto wait_qdo = [&](int t) -> bool {
        return mbar_wait_warp(&qdo_full[t % STAGES], (uint32_t)(t / STAGES) & 1, abort_flag, args.status, ST_TIMEOUT_ATTN);
      };
      auto issue_st = [&](int t) {               // S^T of item t (its Q / dO stage has been waited for)
        const uint64_t q = q_kmaj0 + (uint64_t)((t % STAGES) * TILE16);
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk)
            umma_ss(tmem_base + ST_COL, k_kmaj + KMAJ_STEP(kk), q + KMAJ_STEP(kk), idesc_s, kk > 0 ? 1u : 0u);
          umma_commit(st_full);
        }
      };
      auto issue_dpt = [&](int t) {              // dP^T of item t
        const uint64_t d_o = do_kmaj0 + (uint64_t)((t % STAGES) * TILE16);
        const uint32_t d = tmem_base + DPT_COL + (t % DPT_BUFS) * 128;
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk)
            umma_ss(d, v_kmaj + KMAJ_STEP(kk), d_o + KMAJ_STEP(kk), idesc_s, kk > 0 ? 1u : 0u);
          umma_commit(&dpt_full[t & 1]);
        }
      };
      // column of the packed bf16 operand for contraction step kk (16 queries = 8 columns)
#define PACKED_COL(kk) ((uint32_t)((kk) * 8))
#define P_COL_OF(kk) ((kk) < 4 ? (uint32_t)((kk) * 8) : 64u + (uint32_t)(((kk) - 4) * 8))

      if (ok && n_items > 0) {
        ok = wait_qdo(0);
        if (ok) {
          tc_fence_after_sync();
          issue_st(0);
          issue_dpt(0);
        }
      }
      for (int t = 0; t < n_items && ok; ++t) {
        const int st = t % STAGES;
        const uint64_t q_mn = q_mnmaj0 + (uint64_t)(st * TILE16);
        const uint64_t do_mn = do_mnmaj0 + (uint64_t)(st * TILE16);
        const uint64_t ds_mn = ds_mnmaj0 + (uint64_t)((t % L::DS_BUFS) * DS16);
        const uint32_t dpt = tmem_base + DPT_COL + (t % DPT_BUFS) * 128;
        const uint32_t dq_col = OVERLAP ? (dpt + DQ_IN_DPT) : (tmem_base + ST_COL);
        const uint32_t acc = t > 0 ? 1u : 0u;
        // dV += P^T dO
        if (!mbar_wait_warp(&p_full[t & 1], (uint32_t)(t >> 1) & 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) { ok = false; break; }
        tc_fence_after_sync();
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < ATT_BQ / 16; ++kk)
            umma_ts(tmem_base + DV_COL, tmem_base + ST_COL + P_COL_OF(kk), do_mn + MNMAJ_STEP(kk), idesc_ts,
                    kk > 0 ? 1u : acc);
        }
        if (OVERLAP && t + 1 < n_items) {
          // next item's S^T goes over the region whose P^T the product above consumes (same pipe, in order) and the
          // dS warps have copied to their registers
          if (!wait_qdo(t + 1)) { ok = false; break; }
          if (!mbar_wait_warp(&p_read[t & 1], (uint32_t)(t >> 1) & 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) { ok = false; break; }
          tc_fence_after_sync();
          issue_st(t + 1);
        }
        // dK += dS^T Q ; dQ = dS K
        if (!mbar_wait_warp(&ds_full[t & 1], (uint32_t)(t >> 1) & 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) { ok = false; break; }
        tc_fence_after_sync();
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < ATT_BQ / 16; ++kk)
            umma_ts(tmem_base + DK_COL, dpt + PACKED_COL(kk), q_mn + MNMAJ_STEP(kk), idesc_ts, kk > 0 ? 1u : acc);
#pragma unroll
          for (int kk = 0; kk < ATT_BKV / 16; ++kk)
            umma_ss(dq_col, ds_mn + MNMAJ_STEP(kk), k_mnmaj + MNMAJ_STEP(kk), idesc_dq, kk > 0 ? 1u : 0u);
          umma_commit(&qdo_empty[st]);
          umma_commit(&dq_full[t & 1]);
        }
        if (OVERLAP && t + 1 < n_items) {
          // next item's dP^T goes into the other region once the dQ that lived there (item t-1) has been drained
          if (t >= 1) {
            if (!mbar_wait_warp(&dq_free[(t + 1) & 1], (uint32_t)((t - 1) >> 1) & 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
          }
          issue_dpt(t + 1);
        }
        if (!OVERLAP && t + 1 < n_items) {
          // dQ of this item sits in the S^T region: the next scores wait until it is drained
          if (!mbar_wait_warp(&dq_free[t & 1], (uint32_t)(t >> 1) & 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) { ok = false; break; }
          if (!wait_qdo(t + 1)) { ok = false; break; }
          tc_fence_after_sync();
          issue_st(t + 1);
          issue_dpt(t + 1);
        }
      }
#undef KMAJ_STEP
#undef MNMAJ_STEP
#undef PACKED_COL
#undef P_COL_OF
      if (ok && leader) umma_commit(acc_full);
    }
  } else if (warp < 10) {
    // ------------------------------ exponential warps: S^T_t -> P^T_t ---------------------------
    const int quad = warp & 3;
    const int wg = (warp - 2) >> 2;          // column half
    const int r = quad * 32 + lane;          // key row inside the tile = tensor-memory lane
    const uint32_t lane_addr = uint32_t(quad * 32) << 16;
    bool ok = true;
    for (int t = 0; t < n_items && ok; ++t) {
      const bool diag = (t % n_i) == 0;        // i == j
      if (!mbar_wait(st_full, (uint32_t)t & 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) { ok = false; break; }
      // (the item's Q / dO stage, which carries lse2, arrived before the MMA warp could issue S^T)
      const float* lse = reinterpret_cast<const float*>(smem + L::STAT_OFF + (t % STAGES) * 1024) + wg * 64;
      tc_fence_after_sync();
      const uint32_t s_addr = tmem_base + ST_COL + lane_addr + wg * 64;
      const float2 sc2 = make_float2(args.scale_log2, args.scale_log2);
      uint32_t pk[32], sa[32], sb[32];
      tmem_ld_32x32b_x32(s_addr, sa);
      tmem_ld_32x32b_x32(s_addr + 32, sb);
      tmem_wait_ld();
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t(&sv)[32] = cc ? sb : sa;
        if (diag) {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if ((wg * 64 + cc * 32 + e) < r) sv[e] = 0xff800000u;   // query before key: -inf, probability exactly 0
        }
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          const float4 l = *reinterpret_cast<const float4*>(lse + cc * 32 + e);
          const float2 x0 = __ffma2_rn(make_float2(__uint_as_float(sv[e]), __uint_as_float(sv[e + 1])), sc2,
                                       make_float2(-l.x, -l.y));
          const float2 x1 = __ffma2_rn(make_float2(__uint_as_float(sv[e + 2]), __uint_as_float(sv[e + 3])), sc2,
                                       make_float2(-l.z, -l.w));
          pk[cc * 16 + (e >> 1)] = pack_bf16x2(ex2_approx(x0.x), ex2_approx(x0.y));
          pk[cc * 16 + (e >> 1) + 1] = pack_bf16x2(ex2_approx(x1.x), ex2_approx(x1.y));
        }
      }
      // 64 probabilities = 32 columns of bf16 pairs, over the first 32 fp32 columns of this half
      tmem_st_32x32b_x32(tmem_base + ST_COL + lane_addr + wg * 64, pk);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t & 1]);
    }
    // ---- epilogue: dK_j, dV_j (row = key index) ----
    if (ok && mbar_wait(acc_full, 0, abort_flag, args.status, ST_TIMEOUT_ATTN)) {
      tc_fence_after_sync();
      const long long token = (long long)kvrow + r;
      (void)ADANA_IN_RANGE(token, (long long)args.B * args.S);
      __nv_bfloat16* dk_dst = args.dk + (token * args.Hk + hk) * HD;
      __nv_bfloat16* dv_dst = args.dv + token * args.lddv + (long long)hk * args.dv_hstride;
#pragma unroll 1
      for (int c = wg; c < HD / 32; c += 2) {
        uint32_t a[32], bq[32];
        tmem_ld_32x32b_x32(tmem_base + DK_COL + lane_addr + c * 32, a);
        tmem_ld_32x32b_x32(tmem_base + DV_COL + lane_addr + c * 32, bq);
        tmem_wait_ld();
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 x, y;
          x.x = pack_bf16x2(__uint_as_float(a[q4 * 8 + 0]), __uint_as_float(a[q4 * 8 + 1]));
          x.y = pack_bf16x2(__uint_as_float(a[q4 * 8 + 2]), __uint_as_float(a[q4 * 8 + 3]));
          x.z = pack_bf16x2(__uint_as_float(a[q4 * 8 + 4]), __uint_as_float(a[q4 * 8 + 5]));
          x.w = pack_bf16x2(__uint_as_float(a[q4 * 8 + 6]), __uint_as_float(a[q4 * 8 + 7]));
          y.x = pack_bf16x2(__uint_as_float(bq[q4 * 8 + 0]), __uint_as_float(bq[q4 * 8 + 1]));
          y.y = pack_bf16x2(__uint_as_float(bq[q4 * 8 + 2]), __uint_as_float(bq[q4 * 8 + 3]));
          y.z = pack_bf16x2(__uint_as_float(bq[q4 * 8 + 4]), __uint_as_float(bq[q4 * 8 + 5]));
          y.w = pack_bf16x2(__uint_as_float(bq[q4 * 8 + 6]), __uint_as_float(bq[q4 * 8 + 7]));
          *reinterpret_cast<uint4*>(dk_dst + c * 32 + q4 * 8) = x;
          *reinterpret_cast<uint4*>(dv_dst + c * 32 + q4 * 8) = y;
        }
      }
    }
  } else {
    // ------------------------------ dS warps (10..13): P^T_t, dP^T_t -> dS^T_t, then drain dQ_{t-1} ----------
    const int quad = warp & 3;
    const int r = quad * 32 + lane;          // key row (dS), query row (dQ drain)
    const uint32_t lane_addr = uint32_t(quad * 32) << 16;
    uint8_t* sDQw = smem + L::DQ_OFF + (warp - 10) * L::DQ_BOX;
    bool ok = true;
    // dQ_i of item t: tensor memory -> registers -> swizzled fp32 staging rows -> bulk reduce-adds into the fp32
    // accumulation buffer (the adds happen in L2, 128 bytes at a time).  A warp stages and sends its own 32 query
    // rows, 32 columns per box, and has ONE box: a box may be refilled only after the reduce that was sent from it
    // has read it, so the column chunks of an item are drained at different points of the loop (chunks [c0, c1) per
    // call) with other work in between instead of waiting for the copy engine each time.
    auto drain = [&](int t, int c0, int c1, bool last) -> bool {
      const int g = t / n_i, i = j + t % n_i;
      const int hq = hk * G + g;
      if (!mbar_wait(&dq_full[t & 1], (uint32_t)(t >> 1) & 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) return false;
      tc_fence_after_sync();
      const uint32_t dq_col = OVERLAP ? (tmem_base + DPT_COL + (t % DPT_BUFS) * 128 + DQ_IN_DPT) : (tmem_base + ST_COL);
      const int tok0 = b * args.S + i * ATT_BQ + quad * 32;
#pragma unroll 1
      for (int c = c0; c < c1; ++c) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(dq_col + lane_addr + c * 32, o);
        if (lane == 0) tma_wait_group_read0();      // the previous reduce has read the box
        __syncwarp();
        tmem_wait_ld();
#pragma unroll
        for (int u = 0; u < 8; ++u)
          *reinterpret_cast<uint4*>(sDQw + lane * 128 + ((u ^ (lane & 7)) << 4)) =
              make_uint4(o[u * 4], o[u * 4 + 1], o[u * 4 + 2], o[u * 4 + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_reduce_add_3d(&tmDQ, sDQw, c * 32, hq, tok0);
          tma_commit_group();
        }
      }
      if (last) {
        // every dQ column of the item is in registers or on its way: the region may be overwritten
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&dq_free[t & 1]);
      }
      return true;
    };
    constexpr int NCH = HD / 32;         // dQ column chunks of an item
    for (int t = 0; t < n_items && ok; ++t) {
      const float* nd = reinterpret_cast<const float*>(smem + L::STAT_OFF + (t % STAGES) * 1024) + 128;
      uint32_t pk[64];
      if (!mbar_wait(&p_full[t & 1], (uint32_t)(t >> 1) & 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) { ok = false; break; }
      tc_fence_after_sync();
      {
        uint32_t(&lo)[32] = *reinterpret_cast<uint32_t(*)[32]>(&pk[0]);
        uint32_t(&hi)[32] = *reinterpret_cast<uint32_t(*)[32]>(&pk[32]);
        tmem_ld_32x32b_x32(tmem_base + ST_COL + lane_addr, lo);
        tmem_ld_32x32b_x32(tmem_base + ST_COL + lane_addr + 64, hi);
        tmem_wait_ld();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_read[t & 1]);     // the next item's S^T may overwrite the region
      if (OVERLAP && t > 0) {                          // first half of the previous item's dQ
        if (!drain(t - 1, 0, NCH / 2, false)) { ok = false; break; }
      }
      if (!mbar_wait(&dpt_full[t & 1], (uint32_t)(t >> 1) & 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) { ok = false; break; }
      if (t >= L::DS_BUFS) {
        // the shared-memory tile is free once the dQ product that read it (item t - DS_BUFS) has retired
        const int u = t - L::DS_BUFS;
        if (!mbar_wait(&dq_full[u & 1], (uint32_t)(u >> 1) & 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) { ok = false; break; }
      }
      tc_fence_after_sync();
      const uint32_t dpt = tmem_base + DPT_COL + (t % DPT_BUFS) * 128 + lane_addr;
      uint8_t* sDS = smem + L::DS_OFF + (t % L::DS_BUFS) * (ATT_BQ * ATT_BKV * 2);
      const float2 s2 = make_float2(args.scale, args.scale);
      uint32_t da[16], db[16];
      tmem_ld_32x32b_x16(dpt, da);
#pragma unroll
      for (int c = 0; c < 8; ++c) {            // 16 query columns at a time, the next load in flight
        uint32_t(&dv)[16] = (c & 1) ? db : da;
        uint32_t(&nx)[16] = (c & 1) ? da : db;
        tmem_wait_ld();
        if (c < 7) tmem_ld_32x32b_x16(dpt + (c + 1) * 16, nx);
        uint32_t out[8];
#pragma unroll
        for (int e = 0; e < 16; e += 4) {
          const float4 d = *reinterpret_cast<const float4*>(nd + c * 16 + e);
          const float2 t0 = __ffma2_rn(make_float2(__uint_as_float(dv[e]), __uint_as_float(dv[e + 1])), s2,
                                       make_float2(d.x, d.y));
          const float2 t1 = __ffma2_rn(make_float2(__uint_as_float(dv[e + 2]), __uint_as_float(dv[e + 3])), s2,
                                       make_float2(d.z, d.w));
          const float2 g0 = __fmul2_rn(unpack_bf16x2(pk[c * 8 + (e >> 1)]), t0);
          const float2 g1 = __fmul2_rn(unpack_bf16x2(pk[c * 8 + (e >> 1) + 1]), t1);
          out[e >> 1] = pack_bf16x2(g0.x, g0.y);
          out[(e >> 1) + 1] = pack_bf16x2(g1.x, g1.y);
        }
        // bf16 pairs over dP^T columns [8c, 8c+8): all of them were loaded in this or an earlier step
        tmem_st_32x32b_x8(dpt + c * 8, out);
        // the same 16 values in row r of the [keys][queries] tile, 128B-swizzled: 64-column chunk c / 4, two granules
        uint8_t* row = sDS + (c >> 2) * CHUNK_BYTES + r * 128;
        const int g = (c & 3) * 2;
        *reinterpret_cast<uint4*>(row + (((g) ^ (r & 7)) << 4)) = make_uint4(out[0], out[1], out[2], out[3]);
        *reinterpret_cast<uint4*>(row + (((g + 1) ^ (r & 7)) << 4)) = make_uint4(out[4], out[5], out[6], out[7]);
      }
      fence_proxy_async_smem();
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[t & 1]);
      // head_dim 64: one item behind, so that the dK / dQ products of this item run meanwhile; head_dim 128: at once,
      // the next item's S^T waits for this dQ to leave its region
      if (OVERLAP) {
        if (t > 0) ok = drain(t - 1, NCH / 2, NCH, true);
      } else {
        ok = drain(t, 0, NCH, true);
      }
    }
    if (OVERLAP && ok && n_items > 0) ok = drain(n_items - 1, 0, NCH, true);
    if (lane == 0) tma_wait_group_read0();   // staging rows are not needed any more
    __syncwarp();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b, h, s] = mul * sum_d dO[t, h, d] * O[t, h, d] (the backward passes mul = -scale).  HD/8 neighbouring lanes own one (token, head) vector, each
// with one 16-byte load per operand; the sum is a 3- or 4-step shuffle inside the lane group.
template <int HD>
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out,
                                  float* __restrict__ delta, int B, int S, int H, float mul,
                                  float* __restrict__ dq_zero) {
  constexpr int LPV = HD / 8;
  constexpr int VPW = 32 / LPV;
  const int lane = threadIdx.x & 31;
  const int sub = lane % LPV, grp = lane / LPV;
  const long long warp_global = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long total = (long long)B * S * H;
  for (long long base = warp_global * VPW; base < total; base += n_warps * VPW) {
    const long long item = base + grp;
    const bool ok = item < total;
    const long long it = ok ? item : 0;
    const long long off = it * HD + sub * 8;
    const uint4 ua = *reinterpret_cast<const uint4*>(dout + off);
    const uint4 uo = *reinterpret_cast<const uint4*>(out + off);
    if (ok && dq_zero) {        // the fp32 dQ accumulator of the same (token, head) vector starts from zero
      *reinterpret_cast<float4*>(dq_zero + off) = make_float4(0.f, 0.f, 0.f, 0.f);
      *reinterpret_cast<float4*>(dq_zero + off + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const float2 a0 = unpack_bf16x2(ua.x), a1 = unpack_bf16x2(ua.y), a2 = unpack_bf16x2(ua.z), a3 = unpack_bf16x2(ua.w);
    const float2 o0 = unpack_bf16x2(uo.x), o1 = unpack_bf16x2(uo.y), o2 = unpack_bf16x2(uo.z), o3 = unpack_bf16x2(uo.w);
    float acc = a0.x * o0.x + a0.y * o0.y + a1.x * o1.x + a1.y * o1.y + a2.x * o2.x + a2.y * o2.y + a3.x * o3.x + a3.y * o3.y;
#pragma unroll
    for (int o = LPV / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (ok && sub == 0) {
      const long long tok = it / H;
      const int h = (int)(it - tok * H);
      const long long bb = tok / S, s = tok - bb * S;
      delta[(bb * H + h) * S + s] = acc * mul;
    }
  }
}

template <int HD>
static int launch_attn_bwd(const CUtensorMap& tq, const CUtensorMap& tdo, const CUtensorMap& tk,
                           const CUtensorMap& tv, const CUtensorMap& tdq, const AttBwdArgs& a, cudaStream_t st) {
  auto kern = attn_bwd_kernel<HD>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, AttBwdSmem<HD>::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int grid = a.B * a.Hk * (a.S / ATT_BKV);
  kern<<<grid, ATT_BWD_THREADS, AttBwdSmem<HD>::TOTAL, st>>>(tq, tdo, tk, tv, tdq, a);
  return (int)cudaGetLastError();
}

}  // namespace adana

// dout/out [T, Hq*hd] bf16, q [T,Hq,hd], k [T,Hk,hd], v strided as in the forward; lse2 from the
// forward; delta [B,Hq,S] scratch (written here); dq_acc [T,Hq,hd] fp32 is cleared here (by the kernel that computes
// delta, in the same pass) and holds dQ on exit; dk [T,Hk,hd] bf16; dv written at dvbase with row pitch lddv / head pitch dv_hstride.
extern "C" int adana_attn_bwd(const void* dout, const void* q, const void* k, long long ldv, int v_hstride,
                              const void* vbase, const void* out, const float* lse2, float* delta,
                              float* dq_acc, void* dk, long long lddv, int dv_hstride, void* dvbase, int B,
                              int S, int Hq, int Hk, int hd, float scale, int* status, void* stream_) {
  using namespace adana;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (B <= 0 || S <= 0) return 0;
  if ((hd != 64 && hd != 128) || (S % ATT_BQ) != 0 || Hq % Hk != 0) return -1;
  const uint64_t T = (uint64_t)B * S;
  {
    const long long items = (long long)T * Hq;
    long long blocks = (items + 7) / 8;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (hd == 64)
      attn_delta_kernel<64><<<(int)blocks, 256, 0, st>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)out, delta, B, S, Hq, -scale, dq_acc);
    else
      attn_delta_kernel<128><<<(int)blocks, 256, 0, st>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)out, delta, B, S, Hq, -scale, dq_acc);
  }
  CUtensorMap tq, tdo, tk, tv;
  uint32_t box[3] = {64, ATT_BQ, 1};
  {
    uint64_t dims[3] = {(uint64_t)hd, T, (uint64_t)Hq};
    uint64_t str[3] = {1, (uint64_t)Hq * hd, (uint64_t)hd};
    if (encode_tmap_nd(&tq, q, 3, dims, str, box, 2, 1)) return -2;
    if (encode_tmap_nd(&tdo, dout, 3, dims, str, box, 2, 1)) return -3;
  }
  {
    uint64_t dims[3] = {(uint64_t)hd, T, (uint64_t)Hk};
    uint64_t str[3] = {1, (uint64_t)Hk * hd, (uint64_t)hd};
    if (encode_tmap_nd(&tk, k, 3, dims, str, box, 2, 1)) return -4;
    uint64_t strv[3] = {1, (uint64_t)ldv, (uint64_t)v_hstride};
    if (encode_tmap_nd(&tv, vbase, 3, dims, strv, box, 2, 1)) return -5;
  }
  AttBwdArgs a;
  a.lse2 = lse2; a.ndelta = delta; a.dq_acc = dq_acc;
  a.dk = (__nv_bfloat16*)dk; a.dv = (__nv_bfloat16*)dvbase; a.lddv = lddv; a.dv_hstride = dv_hstride;
  a.B = B; a.S = S; a.Hq = Hq; a.Hk = Hk;
  a.scale = scale; a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  CUtensorMap tdq;   // dq_acc [T, Hq, hd] fp32 seen as (hd, Hq, T); one reduce moves a [32 tokens][1 head][32 cols] box
  {
    uint64_t dims[3] = {(uint64_t)hd, (uint64_t)Hq, T};
    uint64_t str[3] = {1, (uint64_t)hd, (uint64_t)Hq * hd};
    uint32_t box[3] = {32, 1, 32};
    if (encode_tmap_nd(&tdq, dq_acc, 3, dims, str, box, 4, 1)) return -6;
  }
  if (hd == 64) return launch_attn_bwd<64>(tq, tdo, tk, tv, tdq, a, st);
  return launch_attn_bwd<128>(tq, tdo, tk, tv, tdq, a, st);
}

ADANA_DBG_BIND(attention)
