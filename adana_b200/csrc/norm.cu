// LayerNorm (weight only, mean-subtracting) and RMSNorm, forward and backward.
// One CTA per row (grid-stride), the row is held in registers between the statistics pass
// and the normalisation pass, fp32 statistics, 16-byte vector loads/stores.
//
//   forward : y = (x - mean) * rstd * w      (RMSNorm: mean = 0, rstd = rsqrt(mean(x^2)+eps))
//   backward: dx = rstd * (g - mean(g) - xhat * mean(g * xhat)),  g = dy * w   (LN)
//             dx = rstd * (g - xhat * mean(g * xhat))                           (RMS)
//             dw = sum_rows dy * xhat   (per-CTA partial rows, reduced by adana_colsum_f32)
//
// Replaces F.layer_norm / the eager RMSNorm chain of the reference
// (src/models/base.py:24-33, src/models/qwen3.py:66-77); the residual-stream gradient is
// accumulated in place (accumulate_dx) so no separate add kernel runs.
#include "api.h"
#include "common.cuh"

namespace adana {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAXV_LIMIT = 8;  // float4 per thread held in registers -> cols <= 8192

template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  uint2 u = *reinterpret_cast<const uint2*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
  return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T>
__device__ __forceinline__ void store4(T* p, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* p, float4 v) {
  *reinterpret_cast<float4*>(p) = v;
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  uint2 u;
  u.x = pack_bf16x2(v.x, v.y);
  u.y = pack_bf16x2(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = u;
}

// One barrier per reduction: every warp leaves its partial in one of two slot rows (alternating, so that the next
// reduction's writes cannot overtake this one's reads) and every thread adds the eight partials itself.
template <int NT>
__device__ __forceinline__ float block_sum_1bar(float v, float (*slots)[NT / 32], int& turn) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) slots[turn][threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int wv = 0; wv < NT / 32; ++wv) t += slots[turn][wv];
  turn = (turn + 1) % 3;
  return t;
}

// NT threads per CTA: 256, or 192 when a row is a multiple of 192 x 4 elements (768, 1536, 2304 columns), so that no lane
// idles in the last pass over the row.
template <typename TX, typename TY, int KIND, int NORM_MAXV, int NT>
__global__ void __launch_bounds__(NT)
norm_fwd_kernel(const TX* __restrict__ x, const float* __restrict__ w, TY* __restrict__ y,
                float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int cols,
                float eps) {
  __shared__ float red[3][NT / 32];
  int turn = 0;
  const int nv = cols >> 2;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const TX* xr = x + (size_t)row * cols;
    float4 v[NORM_MAXV];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nv) {
        v[i] = load4<TX>(xr + c * 4);
        s += (KIND == 0) ? (v[i].x + v[i].y + v[i].z + v[i].w)
                         : (v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w);
      }
    }
    float mean = 0.f, rstd;
    if (KIND == 0) {
      mean = block_sum_1bar<NT>(s, red, turn) / cols;
      float q = 0.f;
#pragma unroll
      for (int i = 0; i < NORM_MAXV; ++i) {
        const int c = threadIdx.x + i * NT;
        if (c < nv) {
          const float a = v[i].x - mean, b = v[i].y - mean, cc = v[i].z - mean, d = v[i].w - mean;
          q += a * a + b * b + cc * cc + d * d;
        }
      }
      rstd = rsqrtf(block_sum_1bar<NT>(q, red, turn) / cols + eps);
    } else {
      rstd = rsqrtf(block_sum_1bar<NT>(s, red, turn) / cols + eps);
    }
    if (threadIdx.x == 0) {
      if (mean_out) mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
    TY* yr = y + (size_t)row * cols;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nv) {
        const float4 ww = *reinterpret_cast<const float4*>(w + c * 4);
        float4 o;
        o.x = (v[i].x - mean) * rstd * ww.x;
        o.y = (v[i].y - mean) * rstd * ww.y;
        o.z = (v[i].z - mean) * rstd * ww.z;
        o.w = (v[i].w - mean) * rstd * ww.w;
        store4<TY>(yr + c * 4, o);
      }
    }
  }
}

// Registers decide how many rows an SM has in flight: only dy, x and the old dx of the row are held across the
// reduction (g and xhat are recomputed after it), which fits three CTAs of 256 threads per SM for cols <= 3072.
template <typename TDY, typename TX, int KIND, int NORM_MAXV, int NT>
__global__ void __launch_bounds__(NT, NORM_MAXV <= 3 ? (NT == 192 ? 4 : 3) : 1)
norm_bwd_kernel(const TDY* __restrict__ dy, const TX* __restrict__ x, const float* __restrict__ w,
                const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                float* __restrict__ dx, int accumulate_dx, float* __restrict__ dw_partial, int rows,
                int cols, __nv_bfloat16* __restrict__ dx16) {
  // per-row partial sums of the warps, double-buffered by row parity so that one barrier per row
  // separates the writes from the reads and the next row's writes cannot overtake them
  __shared__ float2 red[2][NT / 32];
  const int nv = cols >> 2;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float4 dwacc[NORM_MAXV];
  float4 wreg[NORM_MAXV];
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    dwacc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    const int c = threadIdx.x + i * NT;
    wreg[i] = (c < nv) ? *reinterpret_cast<const float4*>(w + c * 4) : make_float4(0, 0, 0, 0);
  }
  int parity = 0;
  for (int row = blockIdx.x; row < rows; row += gridDim.x, parity ^= 1) {
    const float mean = (KIND == 0) ? mean_in[row] : 0.f;
    const float rstd = rstd_in[row];
    const TDY* dyr = dy + (size_t)row * cols;
    const TX* xr = x + (size_t)row * cols;
    float* dxr = dx + (size_t)row * cols;
    float4 prev[NORM_MAXV];
    // every load of the row is issued before anything waits on one of them
    float4 dv[NORM_MAXV], xv[NORM_MAXV];
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nv) {
        dv[i] = load4<TDY>(dyr + c * 4);
        xv[i] = load4<TX>(xr + c * 4);
        if (accumulate_dx) prev[i] = *reinterpret_cast<const float4*>(dxr + c * 4);
      }
    }
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nv) {
        const float4 d = dv[i];
        const float4 xh = make_float4((xv[i].x - mean) * rstd, (xv[i].y - mean) * rstd, (xv[i].z - mean) * rstd,
                                      (xv[i].w - mean) * rstd);
        dwacc[i].x += d.x * xh.x;
        dwacc[i].y += d.y * xh.y;
        dwacc[i].z += d.z * xh.z;
        dwacc[i].w += d.w * xh.w;
        const float4 g = make_float4(d.x * wreg[i].x, d.y * wreg[i].y, d.z * wreg[i].z, d.w * wreg[i].w);
        s1 += g.x + g.y + g.z + g.w;
        s2 += g.x * xh.x + g.y * xh.y + g.z * xh.z + g.w * xh.w;
      }
    }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    if (lane == 0) red[parity][warp] = make_float2(s1, s2);
    __syncthreads();
    float t1 = 0.f, t2 = 0.f;
#pragma unroll
    for (int wv = 0; wv < NT / 32; ++wv) {
      const float2 t = red[parity][wv];
      t1 += t.x;
      t2 += t.y;
    }
    const float m2 = t2 / cols;
    const float m1 = (KIND == 0) ? t1 / cols : 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nv) {
        const float4 d = dv[i];
        const float4 xh = make_float4((xv[i].x - mean) * rstd, (xv[i].y - mean) * rstd, (xv[i].z - mean) * rstd,
                                      (xv[i].w - mean) * rstd);
        float4 o;
        o.x = rstd * (d.x * wreg[i].x - m1 - xh.x * m2);
        o.y = rstd * (d.y * wreg[i].y - m1 - xh.y * m2);
        o.z = rstd * (d.z * wreg[i].z - m1 - xh.z * m2);
        o.w = rstd * (d.w * wreg[i].w - m1 - xh.w * m2);
        if (accumulate_dx) {
          o.x += prev[i].x; o.y += prev[i].y; o.z += prev[i].z; o.w += prev[i].w;
        }
        *reinterpret_cast<float4*>(dxr + c * 4) = o;
        if (dx16) store4<__nv_bfloat16>(dx16 + (size_t)row * cols + c * 4, o);
      }
    }
  }
  if (dw_partial) {
    float* out = dw_partial + (size_t)blockIdx.x * cols;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nv) *reinterpret_cast<float4*>(out + c * 4) = dwacc[i];
    }
  }
}

// out[c] (+)= sum over rows of partial[r][c], in a fixed order (deterministic).  A 32 x 16 CTA owns 32 columns:
// thread (x, y) adds rows y, y + 16, ... of column x, the 16 sums are folded through shared memory.
constexpr int CS_TX = 32, CS_TY = 16;
__global__ void __launch_bounds__(CS_TX * CS_TY)
colsum_kernel(const float* __restrict__ partial, int n_rows, int cols, float* __restrict__ out, int accumulate) {
  __shared__ float red[CS_TY][CS_TX + 1];
  const int c = blockIdx.x * CS_TX + threadIdx.x;
  float s = 0.f;
  if (c < cols) {
#pragma unroll 4
    for (int r = threadIdx.y; r < n_rows; r += CS_TY) s += partial[(size_t)r * cols + c];
  }
  red[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int j = 0; j < CS_TY; ++j) t += red[j][threadIdx.x];
    out[c] = accumulate ? out[c] + t : t;
  }
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                     long long n) {
  const long long i4 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (long long i = i4; i < n; i += stride) {
    if (i + 3 < n) {
      store4<__nv_bfloat16>(dst + i, *reinterpret_cast<const float4*>(src + i));
    } else {
      for (long long j = i; j < n; ++j) dst[j] = __float2bfloat16(src[j]);
    }
  }
}

}  // namespace adana

using namespace adana;

static int norm_grid(int rows, int per_sm) {
  const int cap = 148 * per_sm;
  return rows < cap ? rows : cap;
}

// passes of 192 threads over a row when that divides it exactly and fits three passes, else 0
static int fits_192(int cols) {
  const int nv = cols / 4;
  return (nv % 192 == 0 && nv / 192 >= 1 && nv / 192 <= 3) ? nv / 192 : 0;
}

// number of float4 per thread needed to hold one row in registers
static int maxv_for(int cols) {
  const int need = (cols / 4 + NORM_THREADS - 1) / NORM_THREADS;
  if (need <= 1) return 1;
  if (need <= 2) return 2;
  if (need <= 3) return 3;
  if (need <= 4) return 4;
  return 8;
}

template <typename TX, typename TY, int KIND>
static void launch_norm_fwd(int mv, int grid, cudaStream_t st, const void* x, const float* w, void* y,
                            float* mean, float* rstd, int rows, int cols, float eps) {
#define NF(V) norm_fwd_kernel<TX, TY, KIND, V, NORM_THREADS><<<grid, NORM_THREADS, 0, st>>>((const TX*)x, w, (TY*)y, mean, rstd, rows, cols, eps)
#define NF192(V) norm_fwd_kernel<TX, TY, KIND, V, 192><<<grid, 192, 0, st>>>((const TX*)x, w, (TY*)y, mean, rstd, rows, cols, eps)
  if (int v192 = fits_192(cols)) {
    if (v192 == 1) NF192(1); else if (v192 == 2) NF192(2); else NF192(3);
    return;
  }
  switch (mv) {
    case 1: NF(1); break;
    case 2: NF(2); break;
    case 3: NF(3); break;
    case 4: NF(4); break;
    default: NF(8); break;
  }
#undef NF
#undef NF192
}

template <typename TD, typename TX, int KIND>
static void launch_norm_bwd(int mv, int grid, cudaStream_t st, const void* dy, const void* x, const float* w,
                            const float* mean, const float* rstd, float* dx, int acc, float* dwp, int rows,
                            int cols, void* dx16) {
#define NB(V) norm_bwd_kernel<TD, TX, KIND, V, NORM_THREADS><<<grid, NORM_THREADS, 0, st>>>((const TD*)dy, (const TX*)x, w, mean, rstd, dx, acc, dwp, rows, cols, (__nv_bfloat16*)dx16)
#define NB192(V) norm_bwd_kernel<TD, TX, KIND, V, 192><<<grid, 192, 0, st>>>((const TD*)dy, (const TX*)x, w, mean, rstd, dx, acc, dwp, rows, cols, (__nv_bfloat16*)dx16)
  if (int v192 = fits_192(cols)) {
    if (v192 == 1) NB192(1); else if (v192 == 2) NB192(2); else NB192(3);
    return;
  }
  switch (mv) {
    case 1: NB(1); break;
    case 2: NB(2); break;
    case 3: NB(3); break;
    case 4: NB(4); break;
    default: NB(8); break;
  }
#undef NB
#undef NB192
}

extern "C" int adana_norm_fwd(const void* x, int x_is_bf16, const float* w, void* y,
                              int y_is_bf16, float* mean, float* rstd, int rows, int cols,
                              float eps, int kind, void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (rows <= 0) return 0;
  if ((cols & 3) || cols > NORM_THREADS * 4 * NORM_MAXV_LIMIT) return -1;
  const int mv = maxv_for(cols);
  const int grid = norm_grid(rows, 8);
  using bf = __nv_bfloat16;
  if (kind == 0) {
    if (!x_is_bf16 && y_is_bf16) launch_norm_fwd<float, bf, 0>(mv, grid, st, x, w, y, mean, rstd, rows, cols, eps);
    else if (!x_is_bf16 && !y_is_bf16) launch_norm_fwd<float, float, 0>(mv, grid, st, x, w, y, mean, rstd, rows, cols, eps);
    else if (x_is_bf16 && y_is_bf16) launch_norm_fwd<bf, bf, 0>(mv, grid, st, x, w, y, mean, rstd, rows, cols, eps);
    else return -3;
  } else {
    if (!x_is_bf16 && y_is_bf16) launch_norm_fwd<float, bf, 1>(mv, grid, st, x, w, y, mean, rstd, rows, cols, eps);
    else if (!x_is_bf16 && !y_is_bf16) launch_norm_fwd<float, float, 1>(mv, grid, st, x, w, y, mean, rstd, rows, cols, eps);
    else if (x_is_bf16 && y_is_bf16) launch_norm_fwd<bf, bf, 1>(mv, grid, st, x, w, y, mean, rstd, rows, cols, eps);
    else return -3;
  }
  return (int)cudaGetLastError();
}

extern "C" int adana_norm_bwd(const void* dy, int dy_is_bf16, const void* x, int x_is_bf16,
                              const float* w, const float* mean, const float* rstd, float* dx,
                              int accumulate_dx, float* dw_partial, int n_partial_rows, int rows,
                              int cols, int kind, void* dx_bf16, void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (rows <= 0) return 0;
  if ((cols & 3) || cols > NORM_THREADS * 4 * NORM_MAXV_LIMIT) return -1;
  const int mv = maxv_for(cols);
  int grid = norm_grid(rows, 4);
  if (dw_partial) {
    if (n_partial_rows <= 0) return -2;
    // every CTA writes its partial row, so the grid must equal the number of partial rows
    grid = n_partial_rows;
  }
  using bf = __nv_bfloat16;
  if (kind == 0) {
    if (dy_is_bf16 && !x_is_bf16) launch_norm_bwd<bf, float, 0>(mv, grid, st, dy, x, w, mean, rstd, dx, accumulate_dx, dw_partial, rows, cols, dx_bf16);
    else if (!dy_is_bf16 && !x_is_bf16) launch_norm_bwd<float, float, 0>(mv, grid, st, dy, x, w, mean, rstd, dx, accumulate_dx, dw_partial, rows, cols, dx_bf16);
    else if (dy_is_bf16 && x_is_bf16) launch_norm_bwd<bf, bf, 0>(mv, grid, st, dy, x, w, mean, rstd, dx, accumulate_dx, dw_partial, rows, cols, dx_bf16);
    else return -3;
  } else {
    if (dy_is_bf16 && !x_is_bf16) launch_norm_bwd<bf, float, 1>(mv, grid, st, dy, x, w, mean, rstd, dx, accumulate_dx, dw_partial, rows, cols, dx_bf16);
    else if (!dy_is_bf16 && !x_is_bf16) launch_norm_bwd<float, float, 1>(mv, grid, st, dy, x, w, mean, rstd, dx, accumulate_dx, dw_partial, rows, cols, dx_bf16);
    else if (dy_is_bf16 && x_is_bf16) launch_norm_bwd<bf, bf, 1>(mv, grid, st, dy, x, w, mean, rstd, dx, accumulate_dx, dw_partial, rows, cols, dx_bf16);
    else return -3;
  }
  return (int)cudaGetLastError();
}

extern "C" int adana_colsum_f32(const float* partial, int n_partial_rows, int cols, float* out,
                                int accumulate, void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (cols <= 0) return 0;
  colsum_kernel<<<(cols + CS_TX - 1) / CS_TX, dim3(CS_TX, CS_TY), 0, st>>>(partial, n_partial_rows, cols, out, accumulate);
  return (int)cudaGetLastError();
}

extern "C" int adana_cast_f32_to_bf16(const float* src, void* dst, long long n, void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (n <= 0) return 0;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  cast_f32_bf16_kernel<<<(int)blocks, 256, 0, st>>>(src, (__nv_bfloat16*)dst, n);
  return (int)cudaGetLastError();
}

extern "C" int adana_version(void) { return 1; }

ADANA_DBG_BIND(norm)
