// Embedding gather / scatter-add, the cross-entropy over a chunk of logits, and small
// elementwise helpers (sigmoid output gate of the Qwen3 attention).
#include "api.h"
#include "common.cuh"

namespace adana {

// ------------------------------------------------------------------------------------------
// Embedding: out[t, :] (fp32 residual stream) = table[idx[t], :]; one warp-group per token row.
// Replaces nn.Embedding forward (reference src/models/enoki.py:293).
// ------------------------------------------------------------------------------------------
template <typename TT>
__global__ void embedding_fwd_kernel(const long long* __restrict__ idx, const TT* __restrict__ table,
                                     float* __restrict__ out, int n_tokens, int dim, int vocab) {
  const int nv = dim >> 2;
  for (int t = blockIdx.x; t < n_tokens; t += gridDim.x) {
    long long id = idx[t];
    if (!ADANA_IN_RANGE(id, vocab) || id < 0 || id >= vocab) id = 0;  // out-of-range ids read row 0 instead of faulting
    const TT* src = table + (size_t)id * dim;
    float* dst = out + (size_t)t * dim;
    for (int c = threadIdx.x; c < nv; c += blockDim.x) {
      float4 v;
      if (sizeof(TT) == 4) {
        v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src) + c * 4);
      } else {
        uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(src) + c * 4);
        float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
        v = make_float4(a.x, a.y, b.x, b.y);
      }
      *reinterpret_cast<float4*>(dst + c * 4) = v;
    }
  }
}

// dtable[idx[t], :] += dout[t, :] with vector reductions (red.global.add.v4.f32 on sm_90+).
// Frequent tokens collide; the adds are resolved in L2.  Replaces embedding_dense_backward.
__global__ void embedding_bwd_kernel(const long long* __restrict__ idx, const float* __restrict__ dout,
                                     float* __restrict__ dtable, int n_tokens, int dim, int vocab) {
  const int nv = dim >> 2;
  for (int t = blockIdx.x; t < n_tokens; t += gridDim.x) {
    const long long id = idx[t];
    if (!ADANA_IN_RANGE(id, vocab) || id < 0 || id >= vocab) continue;
    const float* src = dout + (size_t)t * dim;
    float* dst = dtable + (size_t)id * dim;
    for (int c = threadIdx.x; c < nv; c += blockDim.x) {
      const float4 v = *reinterpret_cast<const float4*>(src + c * 4);
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + c * 4), "f"(v.x),
                   "f"(v.y), "f"(v.z), "f"(v.w)
                   : "memory");
    }
  }
}

// ------------------------------------------------------------------------------------------
// Cross entropy (+ z-loss, + accuracy) over a chunk of fp32 logits [rows, vocab], one CTA per
// row.  Pass 1: online max / sum-exp / argmax.  Pass 2: dlogits (bf16) =
//   grad_scale * [ softmax * (1 + 2 z_coeff lse) - onehot(target) ]      (0 for ignored rows)
// The row sums (ce, lse^2, correct, valid) are accumulated into `sums` with one atomic per row.
// Mirrors the chunked loss of the reference (src/models/chunked_loss.py:68-151) without
// materialising more than one chunk of logits; ignore_index = -1.
// ------------------------------------------------------------------------------------------
constexpr int CE_THREADS = 512;

// exp(m - nm) that stays 0 (not NaN) for a lane that has seen no element yet (m = -inf)
__device__ __forceinline__ float rescale(float m, float nm) {
  return m == -INFINITY ? 0.f : __expf(m - nm);
}

__global__ void __launch_bounds__(CE_THREADS)
ce_fwd_bwd_kernel(const float* __restrict__ logits, long long ld, const long long* __restrict__ targets,
                  int rows, int vocab, float z_coeff, float grad_scale,
                  __nv_bfloat16* __restrict__ dlogits, long long ldd, float* __restrict__ sums,
                  float* __restrict__ lse_out) {
  __shared__ float s_max[CE_THREADS / 32];
  __shared__ float s_sum[CE_THREADS / 32];
  __shared__ int s_arg[CE_THREADS / 32];
  __shared__ float s_bcast[3];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nv = vocab >> 2;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* lr = logits + (size_t)row * ld;
    float m = -INFINITY, s = 0.f;
    int arg = 0;
    for (int c = threadIdx.x; c < nv; c += CE_THREADS) {
      const float4 v = *reinterpret_cast<const float4*>(lr + c * 4);
      const float vm = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
      if (vm > m) {
        s *= __expf(m - vm);
        m = vm;
        arg = c * 4 + (v.x == vm ? 0 : (v.y == vm ? 1 : (v.z == vm ? 2 : 3)));
      }
      s += __expf(v.x - m) + __expf(v.y - m) + __expf(v.z - m) + __expf(v.w - m);
    }
    // warp reduce (max, sum, argmax: lowest index wins ties like torch.argmax)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const float os = __shfl_xor_sync(0xffffffffu, s, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      const float nm = fmaxf(m, om);
      s = s * rescale(m, nm) + os * rescale(om, nm);
      if (om > m || (om == m && oa < arg)) arg = oa;
      m = nm;
    }
    __syncthreads();
    if (lane == 0) {
      s_max[warp] = m;
      s_sum[warp] = s;
      s_arg[warp] = arg;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float M = s_max[0], Ssum = s_sum[0];
      int A = s_arg[0];
      for (int w2 = 1; w2 < CE_THREADS / 32; ++w2) {
        const float om = s_max[w2], os = s_sum[w2];
        const int oa = s_arg[w2];
        const float nm = fmaxf(M, om);
        Ssum = Ssum * rescale(M, nm) + os * rescale(om, nm);
        if (om > M || (om == M && oa < A)) A = oa;
        M = nm;
      }
      const float lse = M + __logf(Ssum);
      const long long tgt = targets[row];
      const bool valid = tgt >= 0 && tgt < vocab;
      if (tgt != -1) (void)ADANA_IN_RANGE(tgt, vocab);      // only -1 (ignored) may lie outside the vocabulary
      s_bcast[0] = M;
      s_bcast[1] = lse;
      s_bcast[2] = valid ? 1.f : 0.f;
      if (lse_out) lse_out[row] = lse;
      if (valid) {
        atomicAdd(&sums[0], lse - lr[tgt]);
        atomicAdd(&sums[3], 1.f);
      }
      atomicAdd(&sums[1], lse * lse);
      if (valid && A == (int)tgt) atomicAdd(&sums[2], 1.f);
    }
    __syncthreads();
    if (dlogits) {
      const float lse = s_bcast[1];
      const bool valid = s_bcast[2] != 0.f;
      const long long tgt = targets[row];
      const float ce_scale = valid ? grad_scale : 0.f;
      const float z_scale = grad_scale * 2.f * z_coeff * lse;
      const float pscale = ce_scale + z_scale;
      __nv_bfloat16* dr = dlogits + (size_t)row * ldd;
      for (int c = threadIdx.x; c < nv; c += CE_THREADS) {
        const float4 v = *reinterpret_cast<const float4*>(lr + c * 4);
        float g0 = __expf(v.x - lse) * pscale, g1 = __expf(v.y - lse) * pscale,
              g2 = __expf(v.z - lse) * pscale, g3 = __expf(v.w - lse) * pscale;
        const int base = c * 4;
        if (valid && tgt >= base && tgt < base + 4) {
          const int j = (int)(tgt - base);
          if (j == 0) g0 -= ce_scale; else if (j == 1) g1 -= ce_scale;
          else if (j == 2) g2 -= ce_scale; else g3 -= ce_scale;
        }
        uint2 u;
        u.x = pack_bf16x2(g0, g1);
        u.y = pack_bf16x2(g2, g3);
        *reinterpret_cast<uint2*>(dr + base) = u;
      }
    }
    __syncthreads();
  }
}

// The same loss over bf16 logits (what the bf16 GEMM epilogue writes; also what the reference's autocast
// produces before its fp32 cross-entropy), eight columns per 16-byte access.  `dlogits` may be the logits
// buffer itself: in pass 2 every thread overwrites exactly the eight values it has just read, so the chunk
// of logits turns into the chunk of dlogits in place and no second [rows, vocab] buffer exists.
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

__global__ void __launch_bounds__(CE_THREADS)
ce_fwd_bwd_bf16_kernel(const __nv_bfloat16* logits, long long ld, const long long* __restrict__ targets,
                       int rows, int vocab, float z_coeff, float grad_scale, __nv_bfloat16* dlogits, long long ldd,
                       float* __restrict__ sums, float* __restrict__ lse_out) {
  __shared__ float s_max[CE_THREADS / 32];
  __shared__ float s_sum[CE_THREADS / 32];
  __shared__ int s_arg[CE_THREADS / 32];
  __shared__ float s_bcast[3];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nv = vocab >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* lr = logits + (size_t)row * ld;
    float m = -INFINITY, s = 0.f;
    int arg = 0;
    for (int c = threadIdx.x; c < nv; c += CE_THREADS) {
      float v[8];
      unpack8(*reinterpret_cast<const uint4*>(lr + c * 8), v);
      float vm = v[0];
#pragma unroll
      for (int i = 1; i < 8; ++i) vm = fmaxf(vm, v[i]);
      if (vm > m) {
        s *= __expf(m - vm);
        m = vm;
        int j = 7;
#pragma unroll
        for (int i = 6; i >= 0; --i)
          if (v[i] == vm) j = i;      // lowest index among equal values, like torch.argmax
        arg = c * 8 + j;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) s += __expf(v[i] - m);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const float os = __shfl_xor_sync(0xffffffffu, s, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      const float nm = fmaxf(m, om);
      s = s * rescale(m, nm) + os * rescale(om, nm);
      if (om > m || (om == m && oa < arg)) arg = oa;
      m = nm;
    }
    __syncthreads();
    if (lane == 0) {
      s_max[warp] = m;
      s_sum[warp] = s;
      s_arg[warp] = arg;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float M = s_max[0], Ssum = s_sum[0];
      int A = s_arg[0];
      for (int w2 = 1; w2 < CE_THREADS / 32; ++w2) {
        const float om = s_max[w2], os = s_sum[w2];
        const int oa = s_arg[w2];
        const float nm = fmaxf(M, om);
        Ssum = Ssum * rescale(M, nm) + os * rescale(om, nm);
        if (om > M || (om == M && oa < A)) A = oa;
        M = nm;
      }
      const float lse = M + __logf(Ssum);
      const long long tgt = targets[row];
      const bool valid = tgt >= 0 && tgt < vocab;
      s_bcast[0] = M;
      s_bcast[1] = lse;
      s_bcast[2] = valid ? 1.f : 0.f;
      if (lse_out) lse_out[row] = lse;
      if (valid) {
        atomicAdd(&sums[0], lse - __bfloat162float(lr[tgt]));
        atomicAdd(&sums[3], 1.f);
      }
      atomicAdd(&sums[1], lse * lse);
      if (valid && A == (int)tgt) atomicAdd(&sums[2], 1.f);
    }
    __syncthreads();     // (also orders thread 0's read of lr[tgt] before pass 2 overwrites it in place)
    if (dlogits) {
      const float lse = s_bcast[1];
      const bool valid = s_bcast[2] != 0.f;
      const long long tgt = targets[row];
      const float ce_scale = valid ? grad_scale : 0.f;
      const float pscale = ce_scale + grad_scale * 2.f * z_coeff * lse;
      __nv_bfloat16* dr = dlogits + (size_t)row * ldd;
      for (int c = threadIdx.x; c < nv; c += CE_THREADS) {
        float v[8];
        unpack8(*reinterpret_cast<const uint4*>(lr + c * 8), v);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __expf(v[i] - lse) * pscale;
        const int base = c * 8;
        if (valid && tgt >= base && tgt < base + 8) {
          const int j = (int)(tgt - base);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (i == j) v[i] -= ce_scale;
        }
        uint4 u;
        u.x = pack_bf16x2(v[0], v[1]);
        u.y = pack_bf16x2(v[2], v[3]);
        u.z = pack_bf16x2(v[4], v[5]);
        u.w = pack_bf16x2(v[6], v[7]);
        *reinterpret_cast<uint4*>(dr + base) = u;
      }
    }
    __syncthreads();
  }
}

// out = a * sigmoid(gate) (Qwen3 attention output gate), and its backward.
__global__ void sigmoid_gate_fwd_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ gate,
                                        long long gate_row_stride, int gate_off, int gate_hstride,
                                        __nv_bfloat16* __restrict__ out, long long n_tokens, int H, int hd) {
  const long long total = n_tokens * H * hd / 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long e = i * 2;
    const long long tok = e / (H * hd);
    const int r = (int)(e - tok * H * hd);
    const int h = r / hd, j = r % hd;
    const float2 av = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(a + e));
    const float2 gv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(
        gate + tok * gate_row_stride + gate_off + h * gate_hstride + j));
    *reinterpret_cast<uint32_t*>(out + e) = pack_bf16x2(av.x * sigmoidf_(gv.x), av.y * sigmoidf_(gv.y));
  }
}

__global__ void sigmoid_gate_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ a,
                                        const __nv_bfloat16* __restrict__ gate, long long gate_row_stride,
                                        int gate_off, int gate_hstride, __nv_bfloat16* __restrict__ da,
                                        __nv_bfloat16* __restrict__ dgate_base, long long n_tokens, int H, int hd) {
  const long long total = n_tokens * H * hd / 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long e = i * 2;
    const long long tok = e / (H * hd);
    const int r = (int)(e - tok * H * hd);
    const int h = r / hd, j = r % hd;
    const long long goff = tok * gate_row_stride + gate_off + h * gate_hstride + j;
    const float2 dv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dout + e));
    const float2 av = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(a + e));
    const float2 gv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(gate + goff));
    const float s0 = sigmoidf_(gv.x), s1 = sigmoidf_(gv.y);
    *reinterpret_cast<uint32_t*>(da + e) = pack_bf16x2(dv.x * s0, dv.y * s1);
    *reinterpret_cast<uint32_t*>(dgate_base + goff) =
        pack_bf16x2(dv.x * av.x * s0 * (1.f - s0), dv.y * av.y * s1 * (1.f - s1));
  }
}

}  // namespace adana

using namespace adana;

extern "C" int adana_embedding_fwd(const long long* idx, const void* table, int table_is_bf16,
                                   float* out, int n_tokens, int dim, int vocab, void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (n_tokens <= 0) return 0;
  if (dim & 3) return -1;
  const int grid = n_tokens < 148 * 16 ? n_tokens : 148 * 16;
  if (table_is_bf16)
    embedding_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(idx, (const __nv_bfloat16*)table, out,
                                                              n_tokens, dim, vocab);
  else
    embedding_fwd_kernel<float><<<grid, 256, 0, st>>>(idx, (const float*)table, out, n_tokens, dim, vocab);
  return (int)cudaGetLastError();
}

extern "C" int adana_embedding_bwd(const long long* idx, const float* dout, float* dtable,
                                   int n_tokens, int dim, int vocab, void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (n_tokens <= 0) return 0;
  if (dim & 3) return -1;
  const int grid = n_tokens < 148 * 16 ? n_tokens : 148 * 16;
  embedding_bwd_kernel<<<grid, 256, 0, st>>>(idx, dout, dtable, n_tokens, dim, vocab);
  return (int)cudaGetLastError();
}

extern "C" int adana_ce_fwd_bwd(float* logits, long long ld, const long long* targets, int rows,
                                int vocab, float z_coeff, float grad_scale, void* dlogits_bf16,
                                long long ldd, float* sums, float* lse_out, void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (rows <= 0) return 0;
  if ((vocab & 3) || (ld & 3) || (ldd & 3)) return -1;
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  ce_fwd_bwd_kernel<<<grid, CE_THREADS, 0, st>>>(logits, ld, targets, rows, vocab, z_coeff, grad_scale,
                                                 (__nv_bfloat16*)dlogits_bf16, ldd, sums, lse_out);
  return (int)cudaGetLastError();
}

// bf16 logits [rows, vocab]; `dlogits_bf16` may alias `logits` (in place) or be null (forward only).
extern "C" int adana_ce_fwd_bwd_bf16(void* logits, long long ld, const long long* targets, int rows, int vocab,
                                     float z_coeff, float grad_scale, void* dlogits_bf16, long long ldd, float* sums,
                                     float* lse_out, void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (rows <= 0) return 0;
  if ((vocab & 7) || (ld & 7) || (ldd & 7)) return -1;
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  ce_fwd_bwd_bf16_kernel<<<grid, CE_THREADS, 0, st>>>((const __nv_bfloat16*)logits, ld, targets, rows, vocab, z_coeff,
                                                      grad_scale, (__nv_bfloat16*)dlogits_bf16, ldd, sums, lse_out);
  return (int)cudaGetLastError();
}

extern "C" int adana_sigmoid_gate_fwd(const void* a, const void* gate, long long gate_row_stride,
                                      int gate_off, int gate_hstride, void* out, long long n_tokens,
                                      int H, int hd, void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (n_tokens <= 0) return 0;
  sigmoid_gate_fwd_kernel<<<148 * 8, 256, 0, st>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)gate,
                                                   gate_row_stride, gate_off, gate_hstride,
                                                   (__nv_bfloat16*)out, n_tokens, H, hd);
  return (int)cudaGetLastError();
}

extern "C" int adana_sigmoid_gate_bwd(const void* dout, const void* a, const void* gate,
                                      long long gate_row_stride, int gate_off, int gate_hstride,
                                      void* da, void* dgate_base, long long n_tokens, int H, int hd,
                                      void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (n_tokens <= 0) return 0;
  sigmoid_gate_bwd_kernel<<<148 * 8, 256, 0, st>>>(
      (const __nv_bfloat16*)dout, (const __nv_bfloat16*)a, (const __nv_bfloat16*)gate, gate_row_stride,
      gate_off, gate_hstride, (__nv_bfloat16*)da, (__nv_bfloat16*)dgate_base, n_tokens, H, hd);
  return (int)cudaGetLastError();
}

ADANA_DBG_BIND(misc)
