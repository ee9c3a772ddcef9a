// Fused optimizer step over a flat fp32 shard: ADana / Dana-MK4 / Dana-Star(-MK4) / AdamW.
//
// One pass reads p, g, m, v (, tau) and writes p, m, v (, tau) plus the bf16 copy of the
// updated parameters that the next forward (or the next all-gather) consumes, so the
// optimizer costs one HBM round trip of the state instead of ~25 elementwise launches per
// tensor.  The global-norm clip coefficient is read from device memory, so no host
// synchronisation sits between the gradient reduction and the update.
//
// Math: see adana_b200/optim/logtime.py (parity: reference src/optim/adana.py:82-153,
// src/optim/dana_star_mk4.py:105-205, src/optim/adamw_decaying_wd.py:40-84).
#include "api.h"
#include "common.cuh"

namespace adana {

constexpr int OPT_THREADS = 256;

__device__ __forceinline__ float signf_(float x) { return (x > 0.f) - (x < 0.f); }

template <int KIND, bool HAS_BF16, bool DIAG>
__global__ void __launch_bounds__(OPT_THREADS)
opt_step_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                float* __restrict__ v, float* __restrict__ tau, __nv_bfloat16* __restrict__ p16,
                long long n, const AdanaOptHyper h, const float* __restrict__ clip_coef_ptr,
                float* __restrict__ diag) {
  const float gs = h.grad_scale * (clip_coef_ptr ? *clip_coef_ptr : 1.f);
  const float tpow = (KIND == 0) ? __powf(1.f + h.step, h.one_minus_kappa) : 0.f;
  const float floor_p = 1.f / (1.f + h.step);
  float d_af = 0.f, d_g2 = 0.f, d_mfac = 0.f, d_m2 = 0.f;
  const long long stride = (long long)gridDim.x * OPT_THREADS;
  for (long long i = (long long)blockIdx.x * OPT_THREADS + threadIdx.x; i < n; i += stride) {
    const float gi = g[i] * gs;
    float pi = p[i];
    float mi = m[i], vi = v[i];
    if (KIND == 0 || KIND == 1) {
      mi = mi + h.alpha * (gi - mi);
      vi = vi * (1.f - h.alpha) + h.alpha * gi * gi;
      const float denom = sqrtf(vi) + h.eps;
      float norm, af, mfac, longterm;
      if (KIND == 0) {
        norm = 1.f / denom;
        mfac = fabsf(mi) * norm;
        af = tpow * mfac;
        if (h.clipsnr >= 0.f) af = fminf(af, h.clipsnr);
        longterm = signf_(mi) * af + mi * norm;
      } else {
        float ti = tau[i];
        const float ag = fabsf(gi);
        ti = ti + h.alpha * (ag / (ag + denom) - ti);
        tau[i] = ti;
        const float ct = fminf(ti, 0.5f);
        const float reg = fmaxf(ct / (1.f - ct), floor_p);
        const float eff = fmaxf(ti * h.step, 1.f);
        norm = sqrtf(reg) / denom;
        const float mn = fabsf(mi) * norm;
        mfac = mn / reg;
        af = __powf(eff, h.one_minus_kappa) * mfac;
        if (h.clipsnr >= 0.f) af = fminf(af, h.clipsnr);
        longterm = signf_(mi) * (reg * af + mn);
      }
      pi += (-h.lr) * gi * norm + (-h.lr) * h.gamma3 * longterm;
      pi *= h.wd_factor;
      if (DIAG) {
        d_af += af;
        d_mfac += mfac;
      }
    } else if (KIND == 4 || KIND == 5) {
      // AdEMAMix (src/optim/ademamix.py:31-195): fast EMA m, slow EMA in the tau buffer, Adam second moment;
      // update = (m / bc1 + gamma3 * alpha_t * slow) / (sqrt(v / bc2) + eps).  KIND 4 adds wd * p to the update,
      // KIND 5 multiplies p by the independent (optionally decaying) factor before the step.
      float si = tau[i];
      mi = h.beta1 * mi + (1.f - h.beta1) * gi;
      si = h.beta3 * si + (1.f - h.beta3) * gi;
      vi = h.beta2 * vi + (1.f - h.beta2) * gi * gi;
      tau[i] = si;
      const float denom = sqrtf(vi) / sqrtf(h.bc2) + h.eps;
      float upd = (mi / h.bc1 + h.alpha * h.gamma3 * si) / denom;
      if (KIND == 5) pi *= h.wd_factor;
      else upd += h.wd_coupled * pi;
      pi -= h.lr * upd;
    } else {
      // KIND 2: AdamW (decay before the step, coupled to lr); KIND 3: Adam step, then the
      // independent (optionally decaying) decay factor.
      if (KIND == 2) pi *= h.wd_factor;
      mi = h.beta1 * mi + (1.f - h.beta1) * gi;
      vi = h.beta2 * vi + (1.f - h.beta2) * gi * gi;
      const float denom = sqrtf(vi) / sqrtf(h.bc2) + h.eps;
      pi -= (h.lr / h.bc1) * mi / denom;
      if (KIND == 3) pi *= h.wd_factor;
    }
    if (DIAG) {
      d_g2 += gi * gi;
      d_m2 += mi * mi;
    }
    p[i] = pi;
    m[i] = mi;
    v[i] = vi;
    if (HAS_BF16) p16[i] = __float2bfloat16(pi);
  }
  if (DIAG) {
    __shared__ float red[4][OPT_THREADS / 32];
    float vals[4] = {d_af, d_g2, d_mfac, d_m2};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float w = warp_sum(vals[k]);
      if ((threadIdx.x & 31) == 0) red[k][threadIdx.x >> 5] = w;
    }
    __syncthreads();
    if (threadIdx.x < 4) {
      float s = 0.f;
      for (int w = 0; w < OPT_THREADS / 32; ++w) s += red[threadIdx.x][w];
      atomicAdd(&diag[threadIdx.x], s);
    }
  }
}

__global__ void __launch_bounds__(OPT_THREADS)
sumsq_kernel(const float* __restrict__ x, long long n, float* __restrict__ out) {
  float s = 0.f;
  const long long stride = (long long)gridDim.x * OPT_THREADS;
  for (long long i = (long long)blockIdx.x * OPT_THREADS + threadIdx.x; i < n; i += stride) {
    const float a = x[i];
    s += a * a;
  }
  __shared__ float red[OPT_THREADS / 32];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < OPT_THREADS / 32; ++w) t += red[w];
    atomicAdd(out, t);
  }
}

// clip coefficient from the accumulated squared norm: coef = min(1, max_norm / (norm + 1e-6)),
// also stores the norm itself in out[1] for logging.
__global__ void clip_coef_kernel(const float* __restrict__ sumsq, float norm_scale, float max_norm,
                                 float* __restrict__ out) {
  const float norm = sqrtf(*sumsq) * norm_scale;
  out[0] = max_norm > 0.f ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
  out[1] = norm;
}

}  // namespace adana

using namespace adana;

static int opt_grid(long long n) {
  long long b = (n + OPT_THREADS - 1) / OPT_THREADS;
  const long long cap = 148 * 16;
  return (int)(b < cap ? (b < 1 ? 1 : b) : cap);
}

extern "C" int adana_opt_step(float* p, const float* g, float* m, float* v, float* tau,
                              void* p_bf16, long long n, const AdanaOptHyper* h,
                              const float* clip_coef_ptr, float* diag, void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (n <= 0) return 0;
  const int grid = opt_grid(n);
  __nv_bfloat16* p16 = reinterpret_cast<__nv_bfloat16*>(p_bf16);
  if ((h->kind == 1 || h->kind == 4 || h->kind == 5) && !tau) return -1;
#define OPT_LAUNCH(K, B, D) \
  opt_step_kernel<K, B, D><<<grid, OPT_THREADS, 0, st>>>(p, g, m, v, tau, p16, n, *h, clip_coef_ptr, diag)
#define OPT_KIND(K)                                         \
  if (p16) {                                                \
    if (diag) OPT_LAUNCH(K, true, true);                    \
    else OPT_LAUNCH(K, true, false);                        \
  } else {                                                  \
    if (diag) OPT_LAUNCH(K, false, true);                   \
    else OPT_LAUNCH(K, false, false);                       \
  }
  switch (h->kind) {
    case 0: OPT_KIND(0) break;
    case 1: OPT_KIND(1) break;
    case 2: OPT_KIND(2) break;
    case 3: OPT_KIND(3) break;
    case 4: OPT_KIND(4) break;
    case 5: OPT_KIND(5) break;
    default: return -2;
  }
#undef OPT_KIND
#undef OPT_LAUNCH
  return (int)cudaGetLastError();
}

extern "C" int adana_sumsq_f32(const float* x, long long n, float* out, void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (n <= 0) return 0;
  sumsq_kernel<<<opt_grid(n), OPT_THREADS, 0, st>>>(x, n, out);
  return (int)cudaGetLastError();
}

extern "C" int adana_clip_coef(const float* sumsq, float norm_scale, float max_norm, float* out,
                               void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  clip_coef_kernel<<<1, 1, 0, st>>>(sumsq, norm_scale, max_norm, out);
  return (int)cudaGetLastError();
}

ADANA_DBG_BIND(optim)
