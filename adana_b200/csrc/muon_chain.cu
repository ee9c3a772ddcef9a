// Distributed Muon on flat rank shards, as a chain of kernels over the peer-memory plane:
//
//   muon_momentum        shard-local: buf <- mu buf + g ; ns_in = g + mu buf (Nesterov) or buf, rounded to bf16 into
//                        this rank's part of a symmetric staging buffer, plus per-block partial sums of squares of
//                        every matrix's piece (fixed grid, plain stores: the Frobenius norm is deterministic)
//   muon_pull            the rank that orthogonalises a matrix gathers ITS pieces from the ranks that hold them
//                        (16-byte loads from peer memory, after a bounded wait for their "staged" flags), sums the
//                        partials of all ranks in fixed order and stores X = ns_in / (|ns_in| + eps) in bf16:
//                        gather, norm and scale in one pass, only the bytes of this rank's matrices cross NVLink
//   (Newton-Schulz: tcgen05 GEMMs of gemm_tcgen05.cu, issued by the host between these kernels)
//   muon_push            the orthogonalised matrix goes straight into the staging buffer of the ranks that hold its
//                        elements (16-byte stores to peer memory); a "pushed" flag per unit follows
//   muon_apply           shard-local, after a bounded wait for the owners' flags: decoupled decay and the scaled
//                        update for matrix pieces, AdamW for everything else, and the new bf16 weights stored into
//                        every rank's resident weight buffer (the parameter all-gather is this kernel's epilogue)
//
// With one rank (or replicated weights) the same kernels run with a single "peer": the local buffers.
// Every wait is bounded and reports ST_TIMEOUT_PEER_FLAG through the status word.  Plain loads and stores only.
//
// Replaces what the reference leaves to DTensor redistribution per matmul (src/optim/muon.py:309-320, 365-395) and
// its per-parameter update loop (src/optim/muon.py:519-567).
#include "api.h"
#include "common.cuh"

namespace adana {
namespace muon {

constexpr int MAX_RANKS = 8;
constexpr int PARTS = 16;            // partial sums of squares per (rank, matrix)
struct Ptrs {
  void* p[MAX_RANKS];
};

// One entry per (parameter slot of the unit) x (this rank's shard): the shard-local element range it covers.
struct Seg {
  long long a, b;        // [a, b) in shard coordinates; a is a multiple of 64, b of 8 for matrices (a == b: nothing lives here)
  int kind;              // 0: orthogonalised matrix, 1: AdamW
  int group;             // 0: weight-decayed group, 1: the other
  float shape_factor;    // matrices: matched_rms * sqrt(max(rows, cols))
  int mat;               // matrices: global matrix number (row of the partial-norm table)
};
static_assert(sizeof(Seg) == 32, "the host packs this struct by hand");

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// Bounded wait of the CTA for flags[r] >= seq, r < world.  false: a wait ran out (status set), touch nothing.
__device__ __forceinline__ bool wait_flags(const uint32_t* flags, uint32_t seq, int world, unsigned long long timeout_ns,
                                           int* status) {
  __shared__ int s_ok;
  if (flags == nullptr) return true;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < world) {
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(flags + threadIdx.x) - seq) < 0) {
      if (((++spins) & 0x3f) == 0 && globaltimer_ns() - t0 > timeout_ns) {
        if (status) atomicCAS(status, 0, ST_TIMEOUT_PEER_FLAG);
        s_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  return s_ok != 0;
}

// Deterministic block sum (256 threads): every thread returns the total.
__device__ __forceinline__ float block_sum_256(float v) {
  __shared__ float red[8];
  __shared__ float total;
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    total = t;
  }
  __syncthreads();
  return total;
}

// grid (PARTS, n_segs), 256 threads.  parts[mat * PARTS + blockIdx.x] = this block's sum of squares.
__global__ void __launch_bounds__(256)
muon_momentum_kernel(const float* __restrict__ g, float* __restrict__ buf, __nv_bfloat16* __restrict__ ns_out,
                     const Seg* __restrict__ segs, const float* __restrict__ clip, float gscale, float mu, int nesterov,
                     float* __restrict__ parts) {
  const Seg sg = segs[blockIdx.y];
  if (sg.kind != 0) return;
  const float gs = gscale * (clip ? clip[0] : 1.f);
  float ss = 0.f;
  const long long n8 = (sg.b - sg.a) >> 3;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n8; i += (long long)PARTS * 256) {
    const long long e = sg.a + i * 8;
    if (!ADANA_IN_RANGE(e + 7, sg.b)) continue;
    float gv[8], bv[8];
    *reinterpret_cast<float4*>(gv) = *reinterpret_cast<const float4*>(g + e);
    *reinterpret_cast<float4*>(gv + 4) = *reinterpret_cast<const float4*>(g + e + 4);
    *reinterpret_cast<float4*>(bv) = *reinterpret_cast<const float4*>(buf + e);
    *reinterpret_cast<float4*>(bv + 4) = *reinterpret_cast<const float4*>(buf + e + 4);
    float o[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gk = gv[k] * gs;
      bv[k] = mu * bv[k] + gk;
      o[k] = nesterov ? gk + mu * bv[k] : bv[k];
    }
    *reinterpret_cast<float4*>(buf + e) = *reinterpret_cast<float4*>(bv);
    *reinterpret_cast<float4*>(buf + e + 4) = *reinterpret_cast<float4*>(bv + 4);
    uint4 w;
    w.x = pack_bf16x2(o[0], o[1]); w.y = pack_bf16x2(o[2], o[3]);
    w.z = pack_bf16x2(o[4], o[5]); w.w = pack_bf16x2(o[6], o[7]);
    *reinterpret_cast<uint4*>(ns_out + e) = w;
    // the norm is that of the rounded values, as the reference normalises after the cast
    const float2 r0 = unpack_bf16x2(w.x), r1 = unpack_bf16x2(w.y), r2 = unpack_bf16x2(w.z), r3 = unpack_bf16x2(w.w);
    ss += r0.x * r0.x + r0.y * r0.y + r1.x * r1.x + r1.y * r1.y + r2.x * r2.x + r2.y * r2.y + r3.x * r3.x + r3.y * r3.y;
  }
  const float t = block_sum_256(ss);
  if (threadIdx.x == 0) parts[(long long)sg.mat * PARTS + blockIdx.x] = t;
}

// X[i] = bf16(staged_r[off + i] * scale), r = (off + i) / shard_len, scale = 1 / (sqrt(sum of all partials) + eps)
__global__ void __launch_bounds__(256)
muon_pull_kernel(Ptrs staged, Ptrs parts, int world, long long shard_len, long long off, long long n, int mat, float eps,
                 __nv_bfloat16* __restrict__ X, const uint32_t* flags, uint32_t seq, unsigned long long timeout_ns,
                 int* status) {
  if (!wait_flags(flags, seq, world, timeout_ns, status)) return;
  float v = 0.f;
  if ((int)threadIdx.x < world * PARTS) {
    const int r = threadIdx.x / PARTS, p = threadIdx.x % PARTS;
    v = reinterpret_cast<const float*>(parts.p[r])[(long long)mat * PARTS + p];
  }
  const float scale = 1.f / (sqrtf(block_sum_256(v)) + eps);
  const long long n8 = n >> 3;
  const long long stride = (long long)gridDim.x * 256;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n8; i += stride) {
    const long long e = off + i * 8;
    const int r = (int)(e / shard_len);
    if (!ADANA_IN_RANGE(r, world)) continue;
    const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(staged.p[r]) + e);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    uint4 w;
    w.x = pack_bf16x2(a.x * scale, a.y * scale); w.y = pack_bf16x2(b.x * scale, b.y * scale);
    w.z = pack_bf16x2(c.x * scale, c.y * scale); w.w = pack_bf16x2(d.x * scale, d.y * scale);
    *reinterpret_cast<uint4*>(X + i * 8) = w;
  }
}

// upd_r[off + i] = X[i] on the rank r = (off + i) / shard_len that holds the element
__global__ void __launch_bounds__(256)
muon_push_kernel(const __nv_bfloat16* __restrict__ X, Ptrs upd, int world, long long shard_len, long long off, long long n) {
  const long long n8 = n >> 3;
  const long long stride = (long long)gridDim.x * 256;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n8; i += stride) {
    const long long e = off + i * 8;
    const int r = (int)(e / shard_len);
    if (!ADANA_IN_RANGE(r, world)) continue;
    *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(upd.p[r]) + e) = *reinterpret_cast<const uint4*>(X + i * 8);
  }
}

struct ApplyHyper {
  float lr[2], wd[2];          // per group
  float b1, b2, eps, bias;     // AdamW of the non-matrix parameters: step = lr / bias * m / (eps + sqrt(v))
  float gscale;
};

// grid (blocks, n_segs).  upd: this rank's piece of the orthogonalised updates, shard coordinates.
__global__ void __launch_bounds__(256)
muon_apply_kernel(float* __restrict__ p, const float* __restrict__ g, const __nv_bfloat16* __restrict__ upd,
                  float* __restrict__ m1, float* __restrict__ m2, const Seg* __restrict__ segs, ApplyHyper h,
                  const float* __restrict__ clip, Ptrs weights, int n_dst, long long push_off, const uint32_t* flags,
                  uint32_t seq, int world, unsigned long long timeout_ns, int* status) {
  const Seg sg = segs[blockIdx.y];
  if (sg.a >= sg.b) return;
  if (sg.kind == 0 && !wait_flags(flags, seq, world, timeout_ns, status)) return;
  const float lr = h.lr[sg.group], keep = 1.f - lr * h.wd[sg.group];
  const float adj = lr * sg.shape_factor;
  const float gs = h.gscale * (clip ? clip[0] : 1.f);
  const long long stride = (long long)gridDim.x * 256;
  if (sg.kind == 0) {
    const long long n8 = (sg.b - sg.a) >> 3;
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n8; i += stride) {
      const long long e = sg.a + i * 8;
      const uint4 u = *reinterpret_cast<const uint4*>(upd + e);
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      const float uv[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
      float pv[8];
      *reinterpret_cast<float4*>(pv) = *reinterpret_cast<const float4*>(p + e);
      *reinterpret_cast<float4*>(pv + 4) = *reinterpret_cast<const float4*>(p + e + 4);
#pragma unroll
      for (int k = 0; k < 8; ++k) pv[k] = pv[k] * keep - adj * uv[k];
      *reinterpret_cast<float4*>(p + e) = *reinterpret_cast<float4*>(pv);
      *reinterpret_cast<float4*>(p + e + 4) = *reinterpret_cast<float4*>(pv + 4);
      uint4 w;
      w.x = pack_bf16x2(pv[0], pv[1]); w.y = pack_bf16x2(pv[2], pv[3]);
      w.z = pack_bf16x2(pv[4], pv[5]); w.w = pack_bf16x2(pv[6], pv[7]);
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r)
        if (r < n_dst) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(weights.p[r]) + push_off + e) = w;
    }
  } else {
    // vectors, embeddings, the head: ranges start on a 64-element boundary (slot and shard boundaries) and end anywhere;
    // four elements per thread, then a scalar tail
    const float step = lr / h.bias;
    const long long n4 = (sg.b - sg.a) >> 2;
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n4; i += stride) {
      const long long e = sg.a + i * 4;
      const float4 gv = *reinterpret_cast<const float4*>(g + e);
      float4 a = *reinterpret_cast<const float4*>(m1 + e), b = *reinterpret_cast<const float4*>(m2 + e);
      float4 pv = *reinterpret_cast<const float4*>(p + e);
      const float g4[4] = {gv.x * gs, gv.y * gs, gv.z * gs, gv.w * gs};
      float a4[4] = {a.x, a.y, a.z, a.w}, b4[4] = {b.x, b.y, b.z, b.w}, p4[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        a4[k] += (1.f - h.b1) * (g4[k] - a4[k]);
        b4[k] += (1.f - h.b2) * (g4[k] * g4[k] - b4[k]);
        p4[k] = p4[k] * keep - step * a4[k] / (h.eps + sqrtf(b4[k]));
      }
      *reinterpret_cast<float4*>(m1 + e) = make_float4(a4[0], a4[1], a4[2], a4[3]);
      *reinterpret_cast<float4*>(m2 + e) = make_float4(b4[0], b4[1], b4[2], b4[3]);
      *reinterpret_cast<float4*>(p + e) = make_float4(p4[0], p4[1], p4[2], p4[3]);
      const uint2 w = make_uint2(pack_bf16x2(p4[0], p4[1]), pack_bf16x2(p4[2], p4[3]));
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r)
        if (r < n_dst) *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(weights.p[r]) + push_off + e) = w;
    }
    for (long long e = sg.a + n4 * 4 + (long long)blockIdx.x * 256 + threadIdx.x; e < sg.b; e += stride) {
      const float gk = g[e] * gs;
      const float a = m1[e] + (1.f - h.b1) * (gk - m1[e]);
      const float b = m2[e] + (1.f - h.b2) * (gk * gk - m2[e]);
      m1[e] = a;
      m2[e] = b;
      const float pv = p[e] * keep - step * a / (h.eps + sqrtf(b));
      p[e] = pv;
      const __nv_bfloat16 w = __float2bfloat16(pv);
      for (int r = 0; r < n_dst; ++r) reinterpret_cast<__nv_bfloat16*>(weights.p[r])[push_off + e] = w;
    }
  }
}

static Ptrs make_ptrs(const unsigned long long* v, int n) {
  Ptrs p;
  for (int i = 0; i < MAX_RANKS; ++i) p.p[i] = i < n ? reinterpret_cast<void*>(v[i]) : nullptr;
  return p;
}
static int grid_for(long long items, int cap) {
  const long long b = (items + 255) / 256;
  return (int)(b < 1 ? 1 : (b < cap ? b : cap));
}

}  // namespace muon
}  // namespace adana

using namespace adana::muon;

extern "C" int adana_muon_parts(void) { return PARTS; }

// g, buf: this rank's fp32 shard of the unit; ns_out: where shard element 0 goes in the bf16 staging buffer;
// segs: device array of n_segs entries; parts: this rank's partial-norm table (fp32, PARTS per matrix).
extern "C" int adana_muon_momentum(const float* g, float* buf, void* ns_out, const void* segs, int n_segs,
                                   const float* clip, float gscale, float mu, int nesterov, float* parts, void* stream_) {
  if (n_segs < 0 || !g || !buf || !ns_out || !parts || (n_segs > 0 && !segs)) return -1;
  if ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(buf) | reinterpret_cast<uintptr_t>(ns_out)) & 15) return -1;
  if (n_segs == 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  muon_momentum_kernel<<<dim3(PARTS, n_segs), 256, 0, st>>>(g, buf, reinterpret_cast<__nv_bfloat16*>(ns_out),
                                                            reinterpret_cast<const Seg*>(segs), clip, gscale, mu, nesterov, parts);
  return (int)cudaGetLastError();
}

// staged_ptrs / parts_ptrs: every rank's staging buffer (unit coordinates) and partial-norm table; [off, off + n) is the
// matrix inside the unit; X receives it scaled to unit Frobenius norm.  flags: this rank's "staged" flag slots of the
// unit (nullptr: do not wait).
extern "C" int adana_muon_pull(const unsigned long long* staged_ptrs, const unsigned long long* parts_ptrs, int world,
                               long long shard_len, long long off, long long n, int mat, float eps, void* X,
                               const void* flags, unsigned int seq, unsigned long long timeout_ns, int* status,
                               void* stream_) {
  if (world < 1 || world > MAX_RANKS || shard_len <= 0 || (shard_len & 7) || (off & 7) || (n & 7) || n < 0 || mat < 0 || !X)
    return -1;
  if (off + n > shard_len * world) return -1;
  if (n == 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  muon_pull_kernel<<<grid_for(n / 8, 148 * 4), 256, 0, st>>>(make_ptrs(staged_ptrs, world), make_ptrs(parts_ptrs, world), world,
                                                            shard_len, off, n, mat, eps, reinterpret_cast<__nv_bfloat16*>(X),
                                                            reinterpret_cast<const uint32_t*>(flags), seq, timeout_ns, status);
  return (int)cudaGetLastError();
}

extern "C" int adana_muon_push(const void* X, const unsigned long long* upd_ptrs, int world, long long shard_len,
                               long long off, long long n, void* stream_) {
  if (world < 1 || world > MAX_RANKS || shard_len <= 0 || (shard_len & 7) || (off & 7) || (n & 7) || n < 0 || !X) return -1;
  if (off + n > shard_len * world) return -1;
  if (n == 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  muon_push_kernel<<<grid_for(n / 8, 148 * 4), 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(X), make_ptrs(upd_ptrs, world),
                                                            world, shard_len, off, n);
  return (int)cudaGetLastError();
}

// hyper: 9 floats {lr0, lr1, wd0, wd1, beta1, beta2, eps, bias, gscale}.  weight_ptrs: n_dst bf16 buffers that receive
// the new values at push_off + shard index (n_dst 0: none).  flags: this rank's "pushed" flag slots of the unit.
extern "C" int adana_muon_apply(float* p, const float* g, const void* upd, float* m1, float* m2, const void* segs,
                                int n_segs, const float* hyper, const float* clip, const unsigned long long* weight_ptrs,
                                int n_dst, long long push_off, long long max_seg_len, const void* flags, unsigned int seq,
                                int world, unsigned long long timeout_ns, int* status, void* stream_) {
  if (n_segs < 0 || n_dst < 0 || n_dst > MAX_RANKS || world < 1 || world > MAX_RANKS || !p || !g || !upd || !m1 || !m2 || !hyper)
    return -1;
  if (n_dst > 0 && (!weight_ptrs || (push_off & 7))) return -1;
  if (n_segs == 0) return 0;
  ApplyHyper h;
  h.lr[0] = hyper[0]; h.lr[1] = hyper[1]; h.wd[0] = hyper[2]; h.wd[1] = hyper[3];
  h.b1 = hyper[4]; h.b2 = hyper[5]; h.eps = hyper[6]; h.bias = hyper[7]; h.gscale = hyper[8];
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  const int gx = grid_for(max_seg_len / 8, 148 * 8);
  muon_apply_kernel<<<dim3(gx, n_segs), 256, 0, st>>>(p, g, reinterpret_cast<const __nv_bfloat16*>(upd), m1, m2,
                                                      reinterpret_cast<const Seg*>(segs), h, clip,
                                                      make_ptrs(weight_ptrs ? weight_ptrs : nullptr, weight_ptrs ? n_dst : 0),
                                                      n_dst, push_off, reinterpret_cast<const uint32_t*>(flags), seq, world,
                                                      timeout_ns, status);
  return (int)cudaGetLastError();
}

ADANA_DBG_BIND(muon)
