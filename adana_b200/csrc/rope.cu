// Per-head QK-norm fused with the rotary embedding, forward and backward.
//
// A (token, head) vector of head_dim = 64 or 128 elements is owned by head_dim/8 neighbouring lanes,
// each holding 8 consecutive elements (one 16-byte access), so the interleaved RoPE pairs
// (2i, 2i+1) are lane-local and the norm statistics are a 3- or 4-step shuffle reduction inside the
// lane group.  Reads q and k straight out of the fused projection output (row pitch / head pitch
// multiples of 8 elements), writes rotated q,k as [token, head, hd] bf16.
//
//   q' = rope(norm(q) * wq),  k' = rope(norm(k) * wk)
//   norm kind 0: LayerNorm over head_dim (weight only, eps), 1: RMSNorm, 2: none
//   rope: (x0, x1) -> (x0 cos - x1 sin, x0 sin + x1 cos), angles from a [S, hd/2, 2] fp32 table
//
// The backward recomputes the statistics from the saved projection output (nothing but the
// projection output itself is kept for backward) and writes dq, dk into the projection-gradient
// buffer in the projection's own layout; weight gradients are per-CTA partial rows.
//
// Replaces q_layernorm/k_layernorm + apply_rotary_emb of the reference
// (src/models/enoki.py:42-61,119-124; src/models/qwen3.py:196-210).
#include <cstdlib>

#include "api.h"
#include "common.cuh"

namespace adana {

constexpr int ROPE_THREADS = 256;
constexpr int ROPE_EPL = 8;     // elements per lane: one 16-byte load of bf16
constexpr int ROPE_UNROLL = 3;  // vectors in flight per lane group: hides load latency (12 heads of 64 per pass)

// A (token, head) vector of HD elements is owned by LPV = HD/8 neighbouring lanes (8 for head_dim
// 64, 16 for 128), so a warp works on 32/LPV vectors at a time, every global access is 16 bytes per
// lane, the interleaved RoPE pairs (2i, 2i+1) stay lane-local and a norm statistic costs log2(LPV)
// shuffles shared by all the vectors of the warp.
template <int LPV>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = LPV / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&x)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y; x[4] = c.x; x[5] = c.y; x[6] = d.x; x[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&x)[8]) {
  uint4 u;
  u.x = pack_bf16x2(x[0], x[1]);
  u.y = pack_bf16x2(x[2], x[3]);
  u.z = pack_bf16x2(x[4], x[5]);
  u.w = pack_bf16x2(x[6], x[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ void load8f(const float* p, float (&x)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}

// Work is dealt by token: a warp takes a token, loads the token's (cos, sin) row once, and walks over the token's
// q and k heads VPW * ROPE_UNROLL at a time, so the inner loop has no division and one angle load per token.
struct RopeHead {
  int src;   // element offset of the head inside the token's projection row
  int hh;    // head index inside q or k
  bool isq, ok;
};
__device__ __forceinline__ RopeHead rope_head(int h, int Hq, int Hall, int q_off, int q_hstride, int k_off,
                                              int k_hstride) {
  RopeHead r;
  r.ok = h < Hall;
  const int hc = r.ok ? h : 0;
  r.isq = hc < Hq;
  r.hh = r.isq ? hc : hc - Hq;
  r.src = r.isq ? q_off + r.hh * q_hstride : k_off + r.hh * k_hstride;
  return r;
}

template <int HD, int KIND, int U, int OCC>
__global__ void __launch_bounds__(ROPE_THREADS, OCC)
qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, long long row_stride, int q_off,
                       int q_hstride, int k_off, int k_hstride, const float* __restrict__ wq,
                       const float* __restrict__ wk, const float* __restrict__ freqs,
                       __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_out,
                       long long n_tokens, int S, int Hq, int Hk, float eps) {
  constexpr int LPV = HD / ROPE_EPL;
  constexpr int VPW = 32 / LPV;
    const int lane = threadIdx.x & 31;
  const int sub = lane % LPV, grp = lane / LPV;
  const long long warp_global = ((long long)blockIdx.x * ROPE_THREADS + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * ROPE_THREADS) >> 5;
  float wqr[8], wkr[8];
  if (KIND != 2) {
    load8f(wq + sub * ROPE_EPL, wqr);
    load8f(wk + sub * ROPE_EPL, wkr);
  }
  const int Hall = Hq + Hk;
  for (long long tok = warp_global; tok < n_tokens; tok += n_warps) {
    float cs[8];  // 4 (cos, sin) pairs of this lane's columns at the token's position
    load8f(freqs + (long long)(tok % S) * HD + sub * ROPE_EPL, cs);
    const __nv_bfloat16* row = qkv + tok * row_stride + sub * ROPE_EPL;
    __nv_bfloat16* qo = q_out + tok * Hq * HD + sub * ROPE_EPL;
    __nv_bfloat16* ko = k_out + tok * Hk * HD + sub * ROPE_EPL;
    for (int h0 = 0; h0 < Hall; h0 += VPW * U) {
      float x[U][8];
      RopeHead it[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        it[u] = rope_head(h0 + u * VPW + grp, Hq, Hall, q_off, q_hstride, k_off, k_hstride);
        // (checked build: the last element this lane reads lies inside the token's projection row)
        if (it[u].ok && !ADANA_IN_RANGE(it[u].src + sub * ROPE_EPL + ROPE_EPL - 1, row_stride)) it[u].ok = false;
        load8(row + (it[u].ok ? it[u].src : 0), x[u]);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (KIND != 2) {
          float mean = 0.f;
          if (KIND == 0) {
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) s += x[u][i];
            mean = group_sum<LPV>(s) * (1.f / HD);
          }
          float q = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) q += (x[u][i] - mean) * (x[u][i] - mean);
          const float rstd = rsqrtf(group_sum<LPV>(q) * (1.f / HD) + eps);
#pragma unroll
          for (int i = 0; i < 8; ++i) x[u][i] = (x[u][i] - mean) * rstd * (it[u].isq ? wqr[i] : wkr[i]);
        }
        float o[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float c = cs[2 * i], s = cs[2 * i + 1];
          o[2 * i] = x[u][2 * i] * c - x[u][2 * i + 1] * s;
          o[2 * i + 1] = x[u][2 * i] * s + x[u][2 * i + 1] * c;
        }
        if (it[u].ok) store8((it[u].isq ? qo : ko) + it[u].hh * HD, o);
      }
    }
  }
}

// DQF32: the query gradient arrives in fp32 (straight from the attention backward's reduce-add accumulator, which saves
// the pass that would round it to bf16 first)
template <int HD, int KIND, bool DQF32, int U, int OCC>
__global__ void __launch_bounds__(ROPE_THREADS, OCC)
qknorm_rope_bwd_kernel(const void* __restrict__ dq_, const __nv_bfloat16* __restrict__ dk,
                       const __nv_bfloat16* __restrict__ qkv, long long row_stride, int q_off,
                       int q_hstride, int k_off, int k_hstride, const float* __restrict__ wq,
                       const float* __restrict__ wk, const float* __restrict__ freqs,
                       __nv_bfloat16* __restrict__ dqkv, float* __restrict__ dwq_partial,
                       float* __restrict__ dwk_partial, long long n_tokens, int S, int Hq, int Hk,
                       float eps, long long active_warps) {
  constexpr int LPV = HD / ROPE_EPL;
  constexpr int VPW = 32 / LPV;
  __shared__ float sdw[2][ROPE_THREADS / 32][HD];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int sub = lane % LPV, grp = lane / LPV;
  const long long warp_global = ((long long)blockIdx.x * ROPE_THREADS + threadIdx.x) >> 5;
  float dwq_acc[8], dwk_acc[8], wqr[8], wkr[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) dwq_acc[i] = dwk_acc[i] = 0.f;
  if (KIND != 2) {
    load8f(wq + sub * ROPE_EPL, wqr);
    load8f(wk + sub * ROPE_EPL, wkr);
  }
  const int Hall = Hq + Hk;
  // warps beyond active_warps take no token (their partial rows are zero): the others get equal shares
  for (long long tok = warp_global < active_warps ? warp_global : n_tokens; tok < n_tokens; tok += active_warps) {
    float cs[8];
    load8f(freqs + (long long)(tok % S) * HD + sub * ROPE_EPL, cs);
    const long long row = tok * row_stride + sub * ROPE_EPL;
    const __nv_bfloat16* dqo = reinterpret_cast<const __nv_bfloat16*>(dq_) + tok * Hq * HD + sub * ROPE_EPL;
    const float* dqf = reinterpret_cast<const float*>(dq_) + tok * Hq * HD + sub * ROPE_EPL;
    const __nv_bfloat16* dko = dk + tok * Hk * HD + sub * ROPE_EPL;
    for (int h0 = 0; h0 < Hall; h0 += VPW * U) {
    float x[U][8], d[U][8];
    RopeHead it[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      it[u] = rope_head(h0 + u * VPW + grp, Hq, Hall, q_off, q_hstride, k_off, k_hstride);
      load8(qkv + row + it[u].src, x[u]);
      if (DQF32 && it[u].isq) load8f(dqf + it[u].hh * HD, d[u]);
      else load8((it[u].isq ? dqo : dko) + it[u].hh * HD, d[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      // undo the rotation: gradient w.r.t. the normalised, weighted vector
      float dn[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float c = cs[2 * i], s = cs[2 * i + 1];
        dn[2 * i] = d[u][2 * i] * c + d[u][2 * i + 1] * s;
        dn[2 * i + 1] = -d[u][2 * i] * s + d[u][2 * i + 1] * c;
      }
      float dx[8];
      if (KIND == 2) {
#pragma unroll
        for (int i = 0; i < 8; ++i) dx[i] = dn[i];
      } else {
        float mean = 0.f;
        if (KIND == 0) {
          float s = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) s += x[u][i];
          mean = group_sum<LPV>(s) * (1.f / HD);
        }
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) q += (x[u][i] - mean) * (x[u][i] - mean);
        const float rstd = rsqrtf(group_sum<LPV>(q) * (1.f / HD) + eps);
        float xh[8], g[8], s1 = 0.f, s2 = 0.f;
        const float live = it[u].ok ? 1.f : 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[i] = (x[u][i] - mean) * rstd;
          g[i] = dn[i] * (it[u].isq ? wqr[i] : wkr[i]);
          s1 += g[i];
          s2 += g[i] * xh[i];
          if (it[u].isq) dwq_acc[i] += live * dn[i] * xh[i];
          else dwk_acc[i] += live * dn[i] * xh[i];
        }
        const float m2 = group_sum<LPV>(s2) * (1.f / HD);
        const float m1 = (KIND == 0) ? group_sum<LPV>(s1) * (1.f / HD) : 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) dx[i] = rstd * (g[i] - m1 - xh[i] * m2);
      }
      if (it[u].ok) store8(dqkv + row + it[u].src, dx);
    }
    }
  }
  if (KIND != 2 && dwq_partial) {
    // fold the VPW lane groups of the warp (same columns, different vectors), then the warps
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
      for (int o = LPV; o < 32; o <<= 1) {
        dwq_acc[i] += __shfl_xor_sync(0xffffffffu, dwq_acc[i], o);
        dwk_acc[i] += __shfl_xor_sync(0xffffffffu, dwk_acc[i], o);
      }
    }
    if (grp == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        sdw[0][warp][sub * ROPE_EPL + i] = dwq_acc[i];
        sdw[1][warp][sub * ROPE_EPL + i] = dwk_acc[i];
      }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < 2 * HD; c += ROPE_THREADS) {
      const int which = c / HD, col = c % HD;
      float s = 0.f;
#pragma unroll
      for (int wv = 0; wv < ROPE_THREADS / 32; ++wv) s += sdw[which][wv][col];
      (which == 0 ? dwq_partial : dwk_partial)[(size_t)blockIdx.x * HD + col] = s;
    }
  }
}

// Tuning variants of the two kernels (vectors in flight per lane group, CTAs per SM asked of the compiler), selected by
// ADANA_ROPE_VARIANT for measurements; 0 is what training uses.  Measured at 16384 tokens x 72 heads of 64: forward
// 0.0666 ms with three vectors and four CTAs per SM (64 registers), 0.0738 with three CTAs, 0.0717 with four vectors;
// backward 0.124 ms with three vectors and two CTAs (128 registers), 0.156 / 0.171 ms when squeezed into three CTAs
// (80 registers, spills).
static int rope_variant() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("ADANA_ROPE_VARIANT");
    v = e ? atoi(e) : 0;
  }
  return v;
}

// Every warp takes the same number of tokens (the last ones one fewer at most): how many warps that needs when at
// most max_blocks CTAs may run.
static long long rope_active_warps(long long n_tokens, long long max_blocks) {
  const long long max_warps = max_blocks * (ROPE_THREADS / 32);
  const long long per_warp = (n_tokens + max_warps - 1) / max_warps;
  return (n_tokens + per_warp - 1) / per_warp;
}

}  // namespace adana

using namespace adana;

extern "C" int adana_qknorm_rope_fwd(const void* qkv, long long row_stride, int q_off,
                                     int q_hstride, int k_off, int k_hstride, const float* wq,
                                     const float* wk, const float* freqs, void* q_out, void* k_out,
                                     long long n_tokens, int S, int Hq, int Hk, int hd, float eps,
                                     int kind, void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (n_tokens <= 0) return 0;
  if (hd != 64 && hd != 128) return -1;
  if ((row_stride & 7) || (q_off & 7) || (k_off & 7) || (q_hstride & 7) || (k_hstride & 7)) return -2;  // 16-byte lanes
  const long long blocks = (rope_active_warps(n_tokens, 148 * 8) + ROPE_THREADS / 32 - 1) / (ROPE_THREADS / 32);
  const int variant = rope_variant();
#define RFV(HD_, K_, U_, O_)                                                                 \
  qknorm_rope_fwd_kernel<HD_, K_, U_, O_><<<(int)blocks, ROPE_THREADS, 0, st>>>(             \
      (const __nv_bfloat16*)qkv, row_stride, q_off, q_hstride, k_off, k_hstride, wq, wk, freqs, \
      (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_out, n_tokens, S, Hq, Hk, eps)
#define RF(HD_, K_)                                                                          \
  do {                                                                                       \
    if (variant == 1) RFV(HD_, K_, 3, 3);                                                    \
    else if (variant == 2) RFV(HD_, K_, 4, 3);                                               \
    else RFV(HD_, K_, 3, 4);                                                                 \
  } while (0)
  if (hd == 64) {
    if (kind == 0) RF(64, 0); else if (kind == 1) RF(64, 1); else RF(64, 2);
  } else {
    if (kind == 0) RF(128, 0); else if (kind == 1) RF(128, 1); else RF(128, 2);
  }
#undef RF
#undef RFV
  return (int)cudaGetLastError();
}

extern "C" int adana_qknorm_rope_bwd(const void* dq, const void* dk, const void* qkv,
                                     long long row_stride, int q_off, int q_hstride, int k_off,
                                     int k_hstride, const float* wq, const float* wk,
                                     const float* freqs, void* dqkv, float* dwq_partial,
                                     float* dwk_partial, int n_partial, long long n_tokens, int S,
                                     int Hq, int Hk, int hd, float eps, int kind, int dq_is_f32, void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (n_tokens <= 0) return 0;
  if (hd != 64 && hd != 128) return -1;
  if (kind != 2 && n_partial <= 0) return -3;
  if ((row_stride & 7) || (q_off & 7) || (k_off & 7) || (q_hstride & 7) || (k_hstride & 7)) return -2;
  const int blocks = kind != 2 ? n_partial : 148 * 8;
  const long long active = rope_active_warps(n_tokens, blocks);
  const int variant = rope_variant();
#define RBV(HD_, K_, F_, U_, O_)                                                             \
  qknorm_rope_bwd_kernel<HD_, K_, F_, U_, O_><<<blocks, ROPE_THREADS, 0, st>>>(              \
      dq, (const __nv_bfloat16*)dk, (const __nv_bfloat16*)qkv, row_stride, q_off, q_hstride, k_off, k_hstride, wq, wk, \
      freqs, (__nv_bfloat16*)dqkv, dwq_partial, dwk_partial, n_tokens, S, Hq, Hk, eps, active)
#define RBF(HD_, K_, F_)                                                                     \
  do {                                                                                       \
    if (variant == 1) RBV(HD_, K_, F_, 2, 3);                                                \
    else if (variant == 2) RBV(HD_, K_, F_, 3, 3);                                           \
    else RBV(HD_, K_, F_, 3, 2);                                                             \
  } while (0)
#define RB(HD_, K_)                                                                          \
  do {                                                                                       \
    if (dq_is_f32) RBF(HD_, K_, true);                                                       \
    else RBF(HD_, K_, false);                                                                \
  } while (0)
  if (hd == 64) {
    if (kind == 0) RB(64, 0); else if (kind == 1) RB(64, 1); else RB(64, 2);
  } else {
    if (kind == 0) RB(128, 0); else if (kind == 1) RB(128, 1); else RB(128, 2);
  }
#undef RB
  return (int)cudaGetLastError();
}

ADANA_DBG_BIND(rope)
