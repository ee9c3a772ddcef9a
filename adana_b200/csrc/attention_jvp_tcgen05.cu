// Forward-mode derivative (JVP) of causal self-attention on tcgen05 tensor cores, bf16, head_dim 64 / 128.
//
// Given q, k, v and tangents tq, tk, tv it returns in ONE pass over the keys
//     o  = softmax(c q k^T) v                                   (the primal output)
//     to = d/de o(q + e tq, k + e tk, v + e tv) at e = 0        (its directional derivative)
// With P = softmax(S), S = c q k^T and St = c (tq k^T + q tk^T):
//     Pt = P o (St - mu),  mu_i = sum_j P_ij St_ij,     to = Pt v + P tv = (P o St) v + P tv - mu o
// so, with unnormalised weights p~ = exp2(c' s - m) exactly as in the forward kernel, a CTA keeps four
// running sums per query row (l = sum p~, mu~ = sum p~ st) and two accumulators in tensor memory
//     O  += P~ V            Ot += (P~ o St) V + P~ Vt
// and finishes with  o = O / l,  to = Ot / l - (mu~ / l) o.  The lazy rescale of the forward kernel applies
// unchanged because every sum is linear in p~.
//
// One CTA = one (batch, head, 128-query tile), 1 CTA per SM:
//   warp 0      TMA: Q, Qt once; K_j, Kt_j, V_j, Vt_j through a 2-stage ring
//   warp 1      MMA: S = Q K^T ; St = Qt K^T + Q Kt^T ; O += P V ; Ot += T V + P Vt   (6 chains per key tile;
//               P and T = P o St are read from tensor memory as the A operand)
//   warps 2..5  softmax, one query row per thread
// Key tile: 128 keys at head_dim 64, 64 keys at head_dim 128, so that S, St, O, Ot, P, T fit the 512
// tensor-memory columns (128+128+64+64+64+64 and 64+64+128+128+32+32).
//
// The reference has no kernel for this derivative (its attention is a library call); the oracle and the
// timed comparator are torch.func.jvp over a plain PyTorch attention (ops/attention_native.py).
#include "api.h"
#include "common.cuh"

namespace adana {

constexpr int JVP_BQ = 128;
constexpr int JVP_THREADS = 192;
constexpr int JVP_STAGES = 2;
constexpr float JVP_RESCALE_THRESHOLD = 8.0f;  // log2 units

template <int HD>
struct JvpCfg {
  static constexpr int BKV = HD == 64 ? 128 : 64;
  static constexpr int Q_TILE = JVP_BQ * HD * 2;       // bytes of a [128, HD] bf16 tile
  static constexpr int KV_TILE = BKV * HD * 2;         // bytes of a [BKV, HD] bf16 tile
  static constexpr int Q_OFF = 0;
  static constexpr int QT_OFF = Q_TILE;
  static constexpr int RING_OFF = 2 * Q_TILE;          // per stage: K | Kt | V | Vt
  static constexpr int STAGE_BYTES = 4 * KV_TILE;
  static constexpr int BAR_OFF = RING_OFF + JVP_STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256;
  // tensor-memory columns
  static constexpr uint32_t S_COL = 0;
  static constexpr uint32_t ST_COL = BKV;
  static constexpr uint32_t O_COL = 2 * BKV;
  static constexpr uint32_t OT_COL = O_COL + HD;
  static constexpr uint32_t P_COL = OT_COL + HD;       // BKV/2 columns of packed bf16 pairs
  static constexpr uint32_t T_COL = P_COL + BKV / 2;
  static_assert(T_COL + BKV / 2 <= 512, "tensor memory budget");
};

struct JvpArgs {
  __nv_bfloat16* out;    // [T, Hq*HD]
  __nv_bfloat16* tout;   // [T, Hq*HD]
  int B, S, Hq, Hk;
  float scale, scale_log2;
  int* status;
};

template <int HD>
__global__ void __launch_bounds__(JVP_THREADS, 1)
attn_jvp_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmQt,
                const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmKt,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmVt,
                const JvpArgs args) {
  using C = JvpCfg<HD>;
  constexpr int BKV = C::BKV;
  constexpr int CHUNKS = HD / 64;                  // 64-column (128-byte) chunks per tile row
  constexpr int Q_CHUNK = JVP_BQ * 128;            // bytes of one chunk of a 128-row tile
  constexpr int KV_CHUNK = BKV * 128;

  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::BAR_OFF);
  uint64_t* q_full = bars;                 // [1]
  uint64_t* kv_full = bars + 1;            // [STAGES]
  uint64_t* kv_empty = bars + 3;           // [STAGES]
  uint64_t* s_full = bars + 5;             // [1]  S and St of tile j are complete
  uint64_t* s_empty = bars + 6;            // [1]  softmax holds them in registers
  uint64_t* p_full = bars + 7;             // [1]  P and T of tile j are in tensor memory
  uint64_t* p_empty = bars + 8;            // [1]  the PV chains of tile j retired
  uint64_t* o_full = bars + 9;             // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = args.S / JVP_BQ;
  const int BH = args.B * args.Hq;
  const int qt = n_qt - 1 - (int)(blockIdx.x / BH);   // heaviest query tiles first
  const int bh = (int)(blockIdx.x % BH);
  const int b = bh / args.Hq, h = bh % args.Hq;
  const int hk = h / (args.Hq / args.Hk);
  const int n_kv = (qt + 1) * (JVP_BQ / BKV);          // key tiles up to and including the diagonal
  const int row0 = b * args.S + qt * JVP_BQ;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < JVP_STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_empty, 4);
    mbar_init(p_full, 4);
    mbar_init(p_empty, 1);
    mbar_init(o_full, 1);
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
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, 2 * C::Q_TILE);
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        tma_load_3d(smem + C::Q_OFF + c * Q_CHUNK, &tmQ, q_full, c * 64, row0, h);
        tma_load_3d(smem + C::QT_OFF + c * Q_CHUNK, &tmQt, q_full, c * 64, row0, h);
      }
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        if (!mbar_wait(&kv_empty[stage], phase ^ 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) {
          ok = false;
          break;
        }
        const int kvrow = b * args.S + j * BKV;
        uint8_t* base = smem + C::RING_OFF + stage * C::STAGE_BYTES;
        mbar_expect_tx(&kv_full[stage], C::STAGE_BYTES);
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
          tma_load_3d(base + 0 * C::KV_TILE + c * KV_CHUNK, &tmK, &kv_full[stage], c * 64, kvrow, hk);
          tma_load_3d(base + 1 * C::KV_TILE + c * KV_CHUNK, &tmKt, &kv_full[stage], c * 64, kvrow, hk);
          tma_load_3d(base + 2 * C::KV_TILE + c * KV_CHUNK, &tmV, &kv_full[stage], c * 64, kvrow, hk);
          tma_load_3d(base + 3 * C::KV_TILE + c * KV_CHUNK, &tmVt, &kv_full[stage], c * 64, kvrow, hk);
        }
        if (++stage == JVP_STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();   // let copies in flight land before the CTA exits
        while (globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------------
    // The whole warp runs the loop in lock step and one elected lane issues, so that addresses and descriptors are
    // computed in warp-uniform code (a tcgen05.mma takes them from uniform registers); descriptors are built once
    // and a product adds the 16-byte-unit offset of its contraction step to the address field.
    {
      const bool leader = elect_one();
      const uint32_t tb = __shfl_sync(0xffffffffu, tmem_base, 0);
      constexpr uint32_t idesc_qk = make_idesc_bf16(JVP_BQ, BKV, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(JVP_BQ, HD, false, true);
      const uint64_t q_desc = make_smem_desc_sw128(smem_u32(smem + C::Q_OFF), 16, 1024);
      const uint64_t qt_desc = make_smem_desc_sw128(smem_u32(smem + C::QT_OFF), 16, 1024);
      const uint64_t ring_k0 = make_smem_desc_sw128(smem_u32(smem + C::RING_OFF), 16, 1024);           // K-major view
      const uint64_t ring_mn0 = make_smem_desc_sw128(smem_u32(smem + C::RING_OFF), KV_CHUNK, 1024);    // MN-major view
      constexpr uint32_t STAGE16 = C::STAGE_BYTES >> 4, KVT16 = C::KV_TILE >> 4;
      bool ok = mbar_wait_warp(q_full, 0, abort_flag, args.status, ST_TIMEOUT_ATTN);
      tc_fence_after_sync();
      // O += P V ; Ot += T V + P Vt for key tile jj (its stage is released afterwards)
      auto issue_pv = [&](int jj) -> bool {
        const int st = jj % JVP_STAGES;
        if (!mbar_wait_warp(p_full, (uint32_t)jj & 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) return false;
        tc_fence_after_sync();
        const uint64_t dv0 = ring_mn0 + (uint64_t)(st * STAGE16 + 2 * KVT16);
        const uint64_t dvt0 = ring_mn0 + (uint64_t)(st * STAGE16 + 3 * KVT16);
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < BKV / 16; ++kk) {
            const uint64_t o = (uint64_t)((kk * 2048) >> 4);
            const uint32_t acc = (jj > 0 || kk > 0) ? 1u : 0u;
            umma_ts(tb + C::O_COL, tb + C::P_COL + kk * 8, dv0 + o, idesc_pv, acc);
            umma_ts(tb + C::OT_COL, tb + C::T_COL + kk * 8, dv0 + o, idesc_pv, acc);
            umma_ts(tb + C::OT_COL, tb + C::P_COL + kk * 8, dvt0 + o, idesc_pv, 1u);
          }
          umma_commit(&kv_empty[st]);
          umma_commit(p_empty);
        }
        return true;
      };
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j % JVP_STAGES;
        const uint32_t kvph = (uint32_t)(j / JVP_STAGES) & 1;
        if (!mbar_wait_warp(&kv_full[st], kvph, abort_flag, args.status, ST_TIMEOUT_ATTN) ||
            !mbar_wait_warp(s_empty, ((uint32_t)j & 1) ^ 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint64_t dk0 = ring_k0 + (uint64_t)(st * STAGE16);
        const uint64_t dkt0 = dk0 + (uint64_t)KVT16;
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            // K-major operands: 16 columns of head_dim per step, 64-column chunks Q_CHUNK / KV_CHUNK bytes apart
            const uint64_t oq = (uint64_t)(((kk >> 2) * Q_CHUNK + (kk & 3) * 32) >> 4);
            const uint64_t ok_ = (uint64_t)(((kk >> 2) * KV_CHUNK + (kk & 3) * 32) >> 4);
            umma_ss(tb + C::S_COL, q_desc + oq, dk0 + ok_, idesc_qk, kk > 0 ? 1u : 0u);
            umma_ss(tb + C::ST_COL, qt_desc + oq, dk0 + ok_, idesc_qk, kk > 0 ? 1u : 0u);
            umma_ss(tb + C::ST_COL, q_desc + oq, dkt0 + ok_, idesc_qk, 1u);
          }
          umma_commit(s_full);
        }
        if (j > 0) ok = issue_pv(j - 1);
      }
      if (ok) ok = issue_pv(n_kv - 1);
      if (ok && leader) umma_commit(o_full);
    }
  } else {
    // ------------------------------ softmax + epilogue (warps 2..5) -------------------------
    const int quad = warp & 3;
    const int r = quad * 32 + lane;               // query row inside the tile
    const uint32_t lane_addr = uint32_t(quad * 32) << 16;
    float m_ref = -INFINITY, l_sum = 0.f, mu_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      if (!mbar_wait(s_full, (uint32_t)j & 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int key0 = j * BKV - qt * JVP_BQ;     // column offset of this tile relative to the query tile
      const bool diag = key0 + BKV > 0;           // some key of the tile lies beyond some query row
      uint32_t pk[BKV / 2], tk[BKV / 2];
      float lacc = 0.f, muacc = 0.f, o_factor = 1.f;
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t sv[32], tv[32];
        tmem_ld_32x32b_x32(tmem_base + C::S_COL + lane_addr + c * 32, sv);
        tmem_ld_32x32b_x32(tmem_base + C::ST_COL + lane_addr + c * 32, tv);
        tmem_wait_ld();
        if (diag) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (key0 + c * 32 + i > r) sv[i] = 0xff800000u;   // -inf: weight exactly 0
        }
        float cmax = fmax3(__uint_as_float(sv[0]), __uint_as_float(sv[1]), __uint_as_float(sv[2]));
#pragma unroll
        for (int i = 3; i + 1 < 32; i += 2) cmax = fmax3(cmax, __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
        cmax = fmaxf(cmax, __uint_as_float(sv[31]));
        const float m_c = cmax * args.scale_log2;
        if (m_c > m_ref + JVP_RESCALE_THRESHOLD) {
          const float f = ex2_approx(m_ref - m_c);
          l_sum *= f;
          mu_sum *= f;
          lacc *= f;
          muacc *= f;
          o_factor *= f;
#pragma unroll
          for (int cc = 0; cc < c; ++cc) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float2 pv = unpack_bf16x2(pk[cc * 16 + i]), tw = unpack_bf16x2(tk[cc * 16 + i]);
              pk[cc * 16 + i] = pack_bf16x2(pv.x * f, pv.y * f);
              tk[cc * 16 + i] = pack_bf16x2(tw.x * f, tw.y * f);
            }
          }
          m_ref = m_c;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = ex2_approx(fmaf(__uint_as_float(sv[i]), args.scale_log2, -m_ref));
          const float p1 = ex2_approx(fmaf(__uint_as_float(sv[i + 1]), args.scale_log2, -m_ref));
          // tangent of the scaled scores; masked columns have p = 0 and contribute nothing
          const float t0 = p0 * (__uint_as_float(tv[i]) * args.scale);
          const float t1 = p1 * (__uint_as_float(tv[i + 1]) * args.scale);
          lacc += p0 + p1;
          muacc += t0 + t1;
          pk[c * 16 + (i >> 1)] = pack_bf16x2(p0, p1);
          tk[c * 16 + (i >> 1)] = pack_bf16x2(t0, t1);
        }
      }
      l_sum += lacc;
      mu_sum += muacc;
      const bool grow = o_factor != 1.f;
      // S and St are in registers: the next tile's score chains may overwrite them
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty);
      if (j > 0) {
        // P / T columns and both accumulators are free once the PV chains of tile j-1 retired
        if (!mbar_wait(p_empty, (uint32_t)(j - 1) & 1, abort_flag, args.status, ST_TIMEOUT_ATTN)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (__any_sync(0xffffffffu, grow)) {
#pragma unroll 1
          for (int c = 0; c < 2 * HD / 32; ++c) {   // O and Ot are adjacent: 2*HD columns
            uint32_t o[32];
            tmem_ld_32x32b_x32(tmem_base + C::O_COL + lane_addr + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * o_factor);
            tmem_st_32x32b_x32(tmem_base + C::O_COL + lane_addr + c * 32, o);
          }
          tmem_wait_st();
        }
      }
#pragma unroll
      for (int c = 0; c < BKV / 64; ++c) {
        uint32_t(&pw)[32] = *reinterpret_cast<uint32_t(*)[32]>(&pk[c * 32]);
        uint32_t(&tw)[32] = *reinterpret_cast<uint32_t(*)[32]>(&tk[c * 32]);
        tmem_st_32x32b_x32(tmem_base + C::P_COL + lane_addr + c * 32, pw);
        tmem_st_32x32b_x32(tmem_base + C::T_COL + lane_addr + c * 32, tw);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- epilogue: o = O / l ; to = Ot / l - (mu / l) o ----
    if (ok && mbar_wait(o_full, 0, abort_flag, args.status, ST_TIMEOUT_ATTN)) {
      tc_fence_after_sync();
      const float inv_l = 1.f / l_sum;
      const float mu = mu_sum * inv_l;
      const long long token = (long long)row0 + r;
      const long long off = token * ((long long)args.Hq * HD) + (long long)h * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32], ot[32];
        tmem_ld_32x32b_x32(tmem_base + C::O_COL + lane_addr + c * 32, o);
        tmem_ld_32x32b_x32(tmem_base + C::OT_COL + lane_addr + c * 32, ot);
        tmem_wait_ld();
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint32_t wo[4], wt[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float o0 = __uint_as_float(o[q4 * 8 + 2 * e]) * inv_l, o1 = __uint_as_float(o[q4 * 8 + 2 * e + 1]) * inv_l;
            const float t0 = __uint_as_float(ot[q4 * 8 + 2 * e]) * inv_l - mu * o0;
            const float t1 = __uint_as_float(ot[q4 * 8 + 2 * e + 1]) * inv_l - mu * o1;
            wo[e] = pack_bf16x2(o0, o1);
            wt[e] = pack_bf16x2(t0, t1);
          }
          *reinterpret_cast<uint4*>(args.out + off + c * 32 + q4 * 8) = make_uint4(wo[0], wo[1], wo[2], wo[3]);
          *reinterpret_cast<uint4*>(args.tout + off + c * 32 + q4 * 8) = make_uint4(wt[0], wt[1], wt[2], wt[3]);
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int HD>
static int launch_attn_jvp(const CUtensorMap (&tm)[6], const JvpArgs& a, cudaStream_t st) {
  auto kern = attn_jvp_kernel<HD>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, JvpCfg<HD>::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int grid = a.B * a.Hq * (a.S / JVP_BQ);
  kern<<<grid, JVP_THREADS, JvpCfg<HD>::TOTAL, st>>>(tm[0], tm[1], tm[2], tm[3], tm[4], tm[5], a);
  return (int)cudaGetLastError();
}

}  // namespace adana

using namespace adana;

// q, tq [T, Hq, hd]; k, tk, v, tv [T, Hk, hd]; out, tout [T, Hq*hd]; all contiguous bf16, T = B*S.
extern "C" int adana_attn_jvp(const void* q, const void* tq, const void* k, const void* tk, const void* v,
                              const void* tv, void* out, void* tout, int B, int S, int Hq, int Hk, int hd,
                              float scale, int* status, void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (B <= 0 || S <= 0) return 0;
  if ((hd != 64 && hd != 128) || (S % JVP_BQ) != 0 || Hk <= 0 || Hq % Hk != 0) return -1;
  const uint64_t T = (uint64_t)B * S;
  const uint32_t bkv = hd == 64 ? 128 : 64;
  CUtensorMap tm[6];
  const void* ptr[6] = {q, tq, k, tk, v, tv};
  for (int i = 0; i < 6; ++i) {
    const int H = i < 2 ? Hq : Hk;
    uint64_t dims[3] = {(uint64_t)hd, T, (uint64_t)H};
    uint64_t str[3] = {1, (uint64_t)H * hd, (uint64_t)hd};
    uint32_t box[3] = {64, i < 2 ? (uint32_t)JVP_BQ : bkv, 1};
    if (encode_tmap_nd(&tm[i], ptr[i], 3, dims, str, box, 2, 1)) return -2 - i;
  }
  JvpArgs a;
  a.out = (__nv_bfloat16*)out;
  a.tout = (__nv_bfloat16*)tout;
  a.B = B; a.S = S; a.Hq = Hq; a.Hk = Hk;
  a.scale = scale;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  if (hd == 64) return launch_attn_jvp<64>(tm, a, st);
  return launch_attn_jvp<128>(tm, a, st);
}

ADANA_DBG_BIND(attention_jvp)
