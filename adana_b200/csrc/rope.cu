// Per-head QK-norm fused with the rotary embedding, forward and backward.
//
// One warp owns one (token, head) vector of head_dim = 64 or 128 elements; a lane holds
// head_dim/32 consecutive elements, so the interleaved RoPE pairs (2i, 2i+1) are lane-local and
// the norm statistics are one warp reduction.  Reads q and k straight out of the fused
// projection output (any row pitch / head pitch), writes rotated q,k as [token, head, hd] bf16.
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
#include "api.h"
#include "common.cuh"

namespace adana {

constexpr int ROPE_THREADS = 256;

constexpr int ROPE_UNROLL = 4;  // (token, head) vectors in flight per warp: hides load latency

template <int EPL>
__device__ __forceinline__ void load_vec(const __nv_bfloat16* p, float (&x)[EPL]) {
  if (EPL == 2) {
    const float2 f = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p));
    x[0] = f.x; x[1] = f.y;
  } else {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
    x[0] = a.x; x[1] = a.y; x[EPL - 2] = b.x; x[EPL - 1] = b.y;
  }
}
template <int EPL>
__device__ __forceinline__ void store_vec(__nv_bfloat16* p, const float (&x)[EPL]) {
  if (EPL == 2) {
    *reinterpret_cast<uint32_t*>(p) = pack_bf16x2(x[0], x[1]);
  } else {
    uint2 u;
    u.x = pack_bf16x2(x[0], x[1]);
    u.y = pack_bf16x2(x[EPL - 2], x[EPL - 1]);
    *reinterpret_cast<uint2*>(p) = u;
  }
}

template <int HD, int KIND>
__global__ void __launch_bounds__(ROPE_THREADS)
qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, long long row_stride, int q_off,
                       int q_hstride, int k_off, int k_hstride, const float* __restrict__ wq,
                       const float* __restrict__ wk, const float* __restrict__ freqs,
                       __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_out,
                       long long n_tokens, int S, int Hq, int Hk, float eps) {
  constexpr int EPL = HD / 32;  // elements per lane (2 or 4)
  constexpr int U = ROPE_UNROLL;
  const int lane = threadIdx.x & 31;
  const long long warp_global = ((long long)blockIdx.x * ROPE_THREADS + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * ROPE_THREADS) >> 5;
  const int Hall = Hq + Hk;
  const long long total = n_tokens * Hall;
  float wqr[EPL], wkr[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    wqr[i] = (KIND != 2) ? wq[lane * EPL + i] : 1.f;
    wkr[i] = (KIND != 2) ? wk[lane * EPL + i] : 1.f;
  }
  for (long long base = warp_global * U; base < total; base += n_warps * U) {
    float x[U][EPL];
    float2 cs[U][EPL / 2];
    long long tok[U];
    int hh[U];
    bool isq[U], ok[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long item = base + u;
      ok[u] = item < total;
      const long long it = ok[u] ? item : 0;
      tok[u] = it / Hall;
      const int h = (int)(it - tok[u] * Hall);
      isq[u] = h < Hq;
      hh[u] = isq[u] ? h : h - Hq;
      const __nv_bfloat16* src = qkv + tok[u] * row_stride +
                                 (isq[u] ? q_off + hh[u] * q_hstride : k_off + hh[u] * k_hstride) + lane * EPL;
      load_vec<EPL>(src, x[u]);
      const int pos = (int)(tok[u] % S);
      const float2* fr = reinterpret_cast<const float2*>(freqs) + (long long)pos * (HD / 2) + lane * (EPL / 2);
#pragma unroll
      for (int i = 0; i < EPL / 2; ++i) cs[u][i] = fr[i];
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (KIND != 2) {
        float mean = 0.f;
        if (KIND == 0) {
          float s = 0.f;
#pragma unroll
          for (int i = 0; i < EPL; ++i) s += x[u][i];
          mean = warp_sum(s) * (1.f / HD);
        }
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) q += (x[u][i] - mean) * (x[u][i] - mean);
        const float rstd = rsqrtf(warp_sum(q) * (1.f / HD) + eps);
#pragma unroll
        for (int i = 0; i < EPL; ++i) x[u][i] = (x[u][i] - mean) * rstd * (isq[u] ? wqr[i] : wkr[i]);
      }
      float o[EPL];
#pragma unroll
      for (int i = 0; i < EPL / 2; ++i) {
        const float c = cs[u][i].x, s = cs[u][i].y;
        o[2 * i] = x[u][2 * i] * c - x[u][2 * i + 1] * s;
        o[2 * i + 1] = x[u][2 * i] * s + x[u][2 * i + 1] * c;
      }
      if (ok[u]) {
        __nv_bfloat16* dst = (isq[u] ? q_out + (tok[u] * Hq + hh[u]) * HD : k_out + (tok[u] * Hk + hh[u]) * HD) + lane * EPL;
        store_vec<EPL>(dst, o);
      }
    }
  }
}

template <int HD, int KIND>
__global__ void __launch_bounds__(ROPE_THREADS)
qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dq, const __nv_bfloat16* __restrict__ dk,
                       const __nv_bfloat16* __restrict__ qkv, long long row_stride, int q_off,
                       int q_hstride, int k_off, int k_hstride, const float* __restrict__ wq,
                       const float* __restrict__ wk, const float* __restrict__ freqs,
                       __nv_bfloat16* __restrict__ dqkv, float* __restrict__ dwq_partial,
                       float* __restrict__ dwk_partial, long long n_tokens, int S, int Hq, int Hk,
                       float eps) {
  constexpr int EPL = HD / 32;
  constexpr int U = ROPE_UNROLL;
  __shared__ float sdw[2][ROPE_THREADS / 32][HD];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const long long warp_global = ((long long)blockIdx.x * ROPE_THREADS + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * ROPE_THREADS) >> 5;
  const int Hall = Hq + Hk;
  const long long total = n_tokens * Hall;
  float dwq_acc[EPL], dwk_acc[EPL], wqr[EPL], wkr[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    dwq_acc[i] = dwk_acc[i] = 0.f;
    wqr[i] = (KIND != 2) ? wq[lane * EPL + i] : 1.f;
    wkr[i] = (KIND != 2) ? wk[lane * EPL + i] : 1.f;
  }
  for (long long base = warp_global * U; base < total; base += n_warps * U) {
    float x[U][EPL], d[U][EPL];
    float2 cs[U][EPL / 2];
    long long off[U];
    bool isq[U], ok[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long item = base + u;
      ok[u] = item < total;
      const long long it = ok[u] ? item : 0;
      const long long tok = it / Hall;
      const int h = (int)(it - tok * Hall);
      isq[u] = h < Hq;
      const int hh = isq[u] ? h : h - Hq;
      off[u] = tok * row_stride + (isq[u] ? q_off + hh * q_hstride : k_off + hh * k_hstride) + lane * EPL;
      const __nv_bfloat16* gsrc = (isq[u] ? dq + (tok * Hq + hh) * HD : dk + (tok * Hk + hh) * HD) + lane * EPL;
      load_vec<EPL>(qkv + off[u], x[u]);
      load_vec<EPL>(gsrc, d[u]);
      const int pos = (int)(tok % S);
      const float2* fr = reinterpret_cast<const float2*>(freqs) + (long long)pos * (HD / 2) + lane * (EPL / 2);
#pragma unroll
      for (int i = 0; i < EPL / 2; ++i) cs[u][i] = fr[i];
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      // undo the rotation: gradient w.r.t. the normalised, weighted vector
      float dn[EPL];
#pragma unroll
      for (int i = 0; i < EPL / 2; ++i) {
        const float c = cs[u][i].x, s = cs[u][i].y;
        dn[2 * i] = d[u][2 * i] * c + d[u][2 * i + 1] * s;
        dn[2 * i + 1] = -d[u][2 * i] * s + d[u][2 * i + 1] * c;
      }
      float dx[EPL];
      if (KIND == 2) {
#pragma unroll
        for (int i = 0; i < EPL; ++i) dx[i] = dn[i];
      } else {
        float mean = 0.f;
        if (KIND == 0) {
          float s = 0.f;
#pragma unroll
          for (int i = 0; i < EPL; ++i) s += x[u][i];
          mean = warp_sum(s) * (1.f / HD);
        }
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) q += (x[u][i] - mean) * (x[u][i] - mean);
        const float rstd = rsqrtf(warp_sum(q) * (1.f / HD) + eps);
        float xh[EPL], g[EPL], s1 = 0.f, s2 = 0.f;
        const float live = ok[u] ? 1.f : 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
          xh[i] = (x[u][i] - mean) * rstd;
          g[i] = dn[i] * (isq[u] ? wqr[i] : wkr[i]);
          s1 += g[i];
          s2 += g[i] * xh[i];
          if (isq[u]) dwq_acc[i] += live * dn[i] * xh[i];
          else dwk_acc[i] += live * dn[i] * xh[i];
        }
        const float m2 = warp_sum(s2) * (1.f / HD);
        const float m1 = (KIND == 0) ? warp_sum(s1) * (1.f / HD) : 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) dx[i] = rstd * (g[i] - m1 - xh[i] * m2);
      }
      if (ok[u]) store_vec<EPL>(dqkv + off[u], dx);
    }
  }
  if (KIND != 2 && dwq_partial) {
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      sdw[0][warp][lane * EPL + i] = dwq_acc[i];
      sdw[1][warp][lane * EPL + i] = dwk_acc[i];
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
  if ((row_stride & 3) || (q_off & 3) || (k_off & 3) || (q_hstride & 3) || (k_hstride & 3)) return -2;
  const long long items = n_tokens * (Hq + Hk);
  long long blocks = (items + 8 * ROPE_UNROLL - 1) / (8 * ROPE_UNROLL);
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
#define RF(HD_, K_)                                                                          \
  qknorm_rope_fwd_kernel<HD_, K_><<<(int)blocks, ROPE_THREADS, 0, st>>>(                     \
      (const __nv_bfloat16*)qkv, row_stride, q_off, q_hstride, k_off, k_hstride, wq, wk, freqs, \
      (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_out, n_tokens, S, Hq, Hk, eps)
  if (hd == 64) {
    if (kind == 0) RF(64, 0); else if (kind == 1) RF(64, 1); else RF(64, 2);
  } else {
    if (kind == 0) RF(128, 0); else if (kind == 1) RF(128, 1); else RF(128, 2);
  }
#undef RF
  return (int)cudaGetLastError();
}

extern "C" int adana_qknorm_rope_bwd(const void* dq, const void* dk, const void* qkv,
                                     long long row_stride, int q_off, int q_hstride, int k_off,
                                     int k_hstride, const float* wq, const float* wk,
                                     const float* freqs, void* dqkv, float* dwq_partial,
                                     float* dwk_partial, int n_partial, long long n_tokens, int S,
                                     int Hq, int Hk, int hd, float eps, int kind, void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (n_tokens <= 0) return 0;
  if (hd != 64 && hd != 128) return -1;
  if (kind != 2 && n_partial <= 0) return -3;
  const int blocks = kind != 2 ? n_partial : 148 * 8;
#define RB(HD_, K_)                                                                          \
  qknorm_rope_bwd_kernel<HD_, K_><<<blocks, ROPE_THREADS, 0, st>>>(                          \
      (const __nv_bfloat16*)dq, (const __nv_bfloat16*)dk, (const __nv_bfloat16*)qkv, row_stride, \
      q_off, q_hstride, k_off, k_hstride, wq, wk, freqs, (__nv_bfloat16*)dqkv, dwq_partial,  \
      dwk_partial, n_tokens, S, Hq, Hk, eps)
  if (hd == 64) {
    if (kind == 0) RB(64, 0); else if (kind == 1) RB(64, 1); else RB(64, 2);
  } else {
    if (kind == 0) RB(128, 0); else if (kind == 1) RB(128, 1); else RB(128, 2);
  }
#undef RB
  return (int)cudaGetLastError();
}
