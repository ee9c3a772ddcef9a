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

template <int HD, int KIND>
__global__ void __launch_bounds__(ROPE_THREADS)
qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, long long row_stride, int q_off,
                       int q_hstride, int k_off, int k_hstride, const float* __restrict__ wq,
                       const float* __restrict__ wk, const float* __restrict__ freqs,
                       __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_out,
                       long long n_tokens, int S, int Hq, int Hk, float eps) {
  constexpr int EPL = HD / 32;  // elements per lane (2 or 4)
  const int lane = threadIdx.x & 31;
  const long long warp_global = ((long long)blockIdx.x * ROPE_THREADS + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * ROPE_THREADS) >> 5;
  const int Hall = Hq + Hk;
  const long long total = n_tokens * Hall;
  for (long long item = warp_global; item < total; item += n_warps) {
    const long long tok = item / Hall;
    const int h = (int)(item - tok * Hall);
    const bool is_q = h < Hq;
    const int hh = is_q ? h : h - Hq;
    const __nv_bfloat16* src =
        qkv + tok * row_stride + (is_q ? q_off + hh * q_hstride : k_off + hh * k_hstride) + lane * EPL;
    float x[EPL];
    if (EPL == 2) {
      float2 f = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(src));
      x[0] = f.x; x[1] = f.y;
    } else {
      uint2 u = *reinterpret_cast<const uint2*>(src);
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
      x[0] = a.x; x[1] = a.y; x[EPL - 2] = b.x; x[EPL - 1] = b.y;
    }
    if (KIND != 2) {
      float mean = 0.f;
      if (KIND == 0) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) s += x[i];
        mean = warp_sum(s) * (1.f / HD);
      }
      float q = 0.f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) q += (x[i] - mean) * (x[i] - mean);
      const float rstd = rsqrtf(warp_sum(q) * (1.f / HD) + eps);
      const float* w = (is_q ? wq : wk) + lane * EPL;
#pragma unroll
      for (int i = 0; i < EPL; ++i) x[i] = (x[i] - mean) * rstd * w[i];
    }
    const int pos = (int)(tok % S);
    const float* fr = freqs + ((long long)pos * (HD / 2) + lane * (EPL / 2)) * 2;
    float o[EPL];
#pragma unroll
    for (int i = 0; i < EPL / 2; ++i) {
      const float c = fr[i * 2], s = fr[i * 2 + 1];
      o[2 * i] = x[2 * i] * c - x[2 * i + 1] * s;
      o[2 * i + 1] = x[2 * i] * s + x[2 * i + 1] * c;
    }
    __nv_bfloat16* dst = (is_q ? q_out + (tok * Hq + hh) * HD : k_out + (tok * Hk + hh) * HD) + lane * EPL;
    if (EPL == 2) {
      *reinterpret_cast<uint32_t*>(dst) = pack_bf16x2(o[0], o[1]);
    } else {
      uint2 u;
      u.x = pack_bf16x2(o[0], o[1]);
      u.y = pack_bf16x2(o[EPL - 2], o[EPL - 1]);
      *reinterpret_cast<uint2*>(dst) = u;
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
  __shared__ float sdw[2][ROPE_THREADS / 32][HD];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const long long warp_global = ((long long)blockIdx.x * ROPE_THREADS + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * ROPE_THREADS) >> 5;
  const int Hall = Hq + Hk;
  const long long total = n_tokens * Hall;
  float dwq_acc[EPL], dwk_acc[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) dwq_acc[i] = dwk_acc[i] = 0.f;

  for (long long item = warp_global; item < total; item += n_warps) {
    const long long tok = item / Hall;
    const int h = (int)(item - tok * Hall);
    const bool is_q = h < Hq;
    const int hh = is_q ? h : h - Hq;
    const long long off = tok * row_stride + (is_q ? q_off + hh * q_hstride : k_off + hh * k_hstride) + lane * EPL;
    const __nv_bfloat16* gsrc = (is_q ? dq + (tok * Hq + hh) * HD : dk + (tok * Hk + hh) * HD) + lane * EPL;
    float x[EPL], d[EPL];
    if (EPL == 2) {
      float2 f = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(qkv + off));
      x[0] = f.x; x[1] = f.y;
      float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(gsrc));
      d[0] = g.x; d[1] = g.y;
    } else {
      uint2 u = *reinterpret_cast<const uint2*>(qkv + off);
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
      x[0] = a.x; x[1] = a.y; x[EPL - 2] = b.x; x[EPL - 1] = b.y;
      uint2 gu = *reinterpret_cast<const uint2*>(gsrc);
      float2 ga = unpack_bf16x2(gu.x), gb = unpack_bf16x2(gu.y);
      d[0] = ga.x; d[1] = ga.y; d[EPL - 2] = gb.x; d[EPL - 1] = gb.y;
    }
    // undo the rotation: gradient w.r.t. the normalised, weighted vector
    const int pos = (int)(tok % S);
    const float* fr = freqs + ((long long)pos * (HD / 2) + lane * (EPL / 2)) * 2;
    float dn[EPL];
#pragma unroll
    for (int i = 0; i < EPL / 2; ++i) {
      const float c = fr[i * 2], s = fr[i * 2 + 1];
      dn[2 * i] = d[2 * i] * c + d[2 * i + 1] * s;
      dn[2 * i + 1] = -d[2 * i] * s + d[2 * i + 1] * c;
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
        for (int i = 0; i < EPL; ++i) s += x[i];
        mean = warp_sum(s) * (1.f / HD);
      }
      float q = 0.f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) q += (x[i] - mean) * (x[i] - mean);
      const float rstd = rsqrtf(warp_sum(q) * (1.f / HD) + eps);
      const float* w = (is_q ? wq : wk) + lane * EPL;
      float xh[EPL], g[EPL], s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        xh[i] = (x[i] - mean) * rstd;
        g[i] = dn[i] * w[i];
        s1 += g[i];
        s2 += g[i] * xh[i];
        if (is_q) dwq_acc[i] += dn[i] * xh[i];
        else dwk_acc[i] += dn[i] * xh[i];
      }
      const float m2 = warp_sum(s2) * (1.f / HD);
      const float m1 = (KIND == 0) ? warp_sum(s1) * (1.f / HD) : 0.f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) dx[i] = rstd * (g[i] - m1 - xh[i] * m2);
    }
    __nv_bfloat16* dst = dqkv + off;
    if (EPL == 2) {
      *reinterpret_cast<uint32_t*>(dst) = pack_bf16x2(dx[0], dx[1]);
    } else {
      uint2 u;
      u.x = pack_bf16x2(dx[0], dx[1]);
      u.y = pack_bf16x2(dx[EPL - 2], dx[EPL - 1]);
      *reinterpret_cast<uint2*>(dst) = u;
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
  long long blocks = (items + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
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
