// Peer-memory collectives over NVLink / NVSwitch for the sharded engine, written as plain kernels
// on mapped peer pointers (every rank maps every other rank's arena once at start-up):
//
//   p2p_barrier            flag barrier: write my sequence number into every peer's flag slot, then
//                          wait (bounded) until every slot of my own flag array reached it
//   p2p_reduce_scatter     one-shot pull: my shard of the gradient unit = sum over ranks of their copy
//                          (fp32, 16-byte loads straight from peer memory), fused with the squared-norm
//                          partial that the gradient clip needs
//   p2p_signal             "my copy of unit u is ready": one sequence number stored into a per-unit flag slot of
//                          every peer.  The flagged reduce-scatter / all-reduce below wait (bounded) for the
//                          flags of the ranks they read, so no rank ever waits at a barrier for a rank whose data
//                          it does not need yet, and a fast rank is never held up in the middle of its backward
//   p2p_reduce_scatter_*   the same pull with a bf16 wire format (each rank first rounds its fp32 gradient unit
//                          to a bf16 staging copy, as the reference's FSDP reduces in bf16; sums stay fp32) and
//                          with the flag wait in front; grids are capped at the few CTAs NVLink needs, because
//                          these kernels run beside the backward GEMMs
//   p2p_all_reduce_*       data-parallel (replicated) engines: rank k sums slice k of every rank's unit and stores
//                          the sum into slice k of every rank's fp32 gradient buffer (reduce-scatter and all-gather
//                          in one kernel; slices are disjoint, so it runs in place)
//   p2p_publish_f32        each rank stores one float (its squared-norm partial) into slot [rank] of
//                          every peer: a scalar all-gather; after a barrier everybody sums locally
//   p2p_opt_step_push      the fused optimizer step whose bf16 output is stored directly into every
//                          rank's resident weight buffer: the parameter all-gather is the optimizer's
//                          epilogue, no staging buffer and no separate collective
//
// On a full-bandwidth switch one-shot algorithms are the right shape: every GPU talks to every peer
// directly, nothing is forwarded.  No TMA, no cluster features and no in-switch reduction are used
// here; loads and stores are ordinary global accesses.  Every spin is bounded and reports
// ST_TIMEOUT_PEER_FLAG through the status word instead of hanging.
//
// Replaces the NCCL reduce-scatter / all-gather issued by FSDP2 in the reference
// (src/distributed/fsdp.py:105-116) and the per-tensor optimizer launches (src/optim/adana.py:160-227).
#include <cstdlib>

#include "api.h"
#include "common.cuh"

namespace adana {

constexpr int MAX_RANKS = 8;
struct PeerPtrs {
  void* p[MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys_u32(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// flags.p[r] = base of rank r's flag array (uint32 slots).  Thread t < world talks to peer t.
__global__ void p2p_barrier_kernel(PeerPtrs flags, int rank, int world, int slot_base, uint32_t seq,
                                   unsigned long long timeout_ns, int* status) {
  const int t = threadIdx.x;
  if (t >= world) return;
  __threadfence_system();
  st_release_sys_u32(reinterpret_cast<uint32_t*>(flags.p[t]) + slot_base + rank, seq);
  const uint32_t* mine = reinterpret_cast<const uint32_t*>(flags.p[rank]) + slot_base + t;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  // sequence numbers only grow; compare with wrap-around in mind
  while ((int32_t)(ld_acquire_sys_u32(mine) - seq) < 0) {
    if (((++spins) & 0x3f) == 0 && globaltimer_ns() - t0 > timeout_ns) {
      if (status) atomicCAS(status, 0, ST_TIMEOUT_PEER_FLAG);
      return;
    }
  }
}

// out[i] = sum_r grads_r[shard_off + i], sumsq += sum out[i]^2      (n multiple of 4)
__global__ void __launch_bounds__(256)
p2p_reduce_scatter_kernel(PeerPtrs grads, int world, long long shard_off, long long n, float* __restrict__ out,
                          float* __restrict__ sumsq) {
  float ss = 0.f;
  const long long nv = n >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r) {
      if (r < world) {
        const float4 v = *(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + shard_off) + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
    }
    reinterpret_cast<float4*>(out)[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  if (sumsq) {
    __shared__ float red[8];
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < 8; ++w) t += red[w];
      atomicAdd(sumsq, t);
    }
  }
}

// flags.p[t] + slot + rank <- seq on every rank t (release: everything this rank wrote before is visible first)
__global__ void p2p_signal_kernel(PeerPtrs flags, int rank, int world, int slot, uint32_t seq) {
  const int t = threadIdx.x;
  if (t >= world) return;
  __threadfence_system();
  st_release_sys_u32(reinterpret_cast<uint32_t*>(flags.p[t]) + slot + rank, seq);
}

// Bounded wait of a CTA for the flags of ranks [0, world): my_flags[r] >= seq.  Returns false when a wait ran out
// (status word set): the caller then leaves its output untouched.
__device__ __forceinline__ bool wait_unit_flags(const uint32_t* my_flags, uint32_t seq, int world,
                                                unsigned long long timeout_ns, int* status) {
  __shared__ int s_ok;
  if (my_flags == nullptr) return true;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < world) {
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys_u32(my_flags + threadIdx.x) - seq) < 0) {
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

__device__ __forceinline__ void add8(float (&acc)[8], const uint4& u) {
  const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
}

// Sum over ranks of 8 consecutive elements starting at element `e` of every rank's buffer (fp32 or bf16 wire),
// ranks in fixed order: every rank computes bitwise the same sums.
template <bool BF16>
__device__ __forceinline__ void pull8(const PeerPtrs& src, int world, long long e, float (&acc)[8]) {
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  if (BF16) {
    uint4 u[MAX_RANKS];
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r)
      if (r < world) u[r] = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(src.p[r]) + e);
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r)
      if (r < world) add8(acc, u[r]);
  } else {
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r) {
      if (r < world) {
        const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src.p[r]) + e);
        const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src.p[r]) + e + 4);
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
        acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
      }
    }
  }
}

__device__ __forceinline__ void block_add_to(float* dst, float v) {
  __shared__ float red[8];
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    atomicAdd(dst, t);
  }
}

// out[i] = sum_r src_r[shard_off + i] (fp32), sumsq += sum out[i]^2, after every rank's flag for the unit arrived.
// n and shard_off are multiples of 8.
template <bool BF16>
__global__ void __launch_bounds__(256)
p2p_reduce_scatter_flag_kernel(PeerPtrs src, const uint32_t* my_flags, uint32_t seq, int world, long long shard_off,
                               long long n, float* __restrict__ out, float* __restrict__ sumsq,
                               unsigned long long timeout_ns, int* status) {
  if (!wait_unit_flags(my_flags, seq, world, timeout_ns, status)) return;
  float ss = 0.f;
  const long long n8 = n >> 3;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
    float acc[8];
    pull8<BF16>(src, world, shard_off + i * 8, acc);
    *reinterpret_cast<float4*>(out + i * 8) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(out + i * 8 + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += acc[k] * acc[k];
  }
  if (sumsq) block_add_to(sumsq, ss);
}

// dst_r[slice_off + i] = sum_q src_q[slice_off + i] on EVERY rank r (fp32 destinations): all-reduce of one slice.
template <bool BF16>
__global__ void __launch_bounds__(256)
p2p_all_reduce_flag_kernel(PeerPtrs src, PeerPtrs dst, const uint32_t* my_flags, uint32_t seq, int world,
                           long long slice_off, long long n, float* __restrict__ sumsq, unsigned long long timeout_ns,
                           int* status) {
  if (!wait_unit_flags(my_flags, seq, world, timeout_ns, status)) return;
  float ss = 0.f;
  const long long n8 = n >> 3;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
    float acc[8];
    const long long e = slice_off + i * 8;
    pull8<BF16>(src, world, e, acc);
    const float4 lo = make_float4(acc[0], acc[1], acc[2], acc[3]), hi = make_float4(acc[4], acc[5], acc[6], acc[7]);
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r) {
      if (r < world) {
        float* d = reinterpret_cast<float*>(dst.p[r]) + e;
        *reinterpret_cast<float4*>(d) = lo;
        *reinterpret_cast<float4*>(d + 4) = hi;
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += acc[k] * acc[k];
  }
  // squared norm of this rank's slice of the reduced gradient: the ranks publish these partials and add them in rank
  // order, so every rank derives bitwise the same clip coefficient
  if (sumsq) block_add_to(sumsq, ss);
}

__global__ void p2p_publish_f32_kernel(PeerPtrs slots, int rank, int world, const float* __restrict__ value) {
  const int t = threadIdx.x;
  if (t < world) reinterpret_cast<float*>(slots.p[t])[rank] = *value;
}

// coef = min(1, max_norm / (norm + 1e-6)) from the per-rank squared-norm partials
__global__ void clip_coef_multi_kernel(const float* __restrict__ partials, int world, float norm_scale, float max_norm,
                                       float* __restrict__ out) {
  float s = 0.f;
  for (int r = 0; r < world; ++r) s += partials[r];
  const float norm = sqrtf(s) * norm_scale;
  out[0] = max_norm > 0.f ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
  out[1] = norm;
}

// dst_r[dst_off + i] = src[i] on every rank r (fp32; the exact copy of the small norm weights)
__global__ void p2p_push_f32_kernel(const float* __restrict__ src, PeerPtrs dst, int world, long long dst_off,
                                    long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float v = src[i];
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r)
      if (r < world) reinterpret_cast<float*>(dst.p[r])[dst_off + i] = v;
  }
}

__device__ __forceinline__ float sgn(float x) { return (x > 0.f) - (x < 0.f); }

// Fused optimizer step (same math as optim.cu) over [0, n) of a flat shard, 8 elements per thread;
// the bf16 result of element i is stored at weights_r[push_off + i] on every rank r.
template <int KIND>
__global__ void __launch_bounds__(256)
p2p_opt_step_push_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                         float* __restrict__ tau, PeerPtrs weights, int world, long long push_off, long long n,
                         const AdanaOptHyper h, const float* __restrict__ clip_coef_ptr) {
  const float gs = h.grad_scale * (clip_coef_ptr ? *clip_coef_ptr : 1.f);
  const float tpow = (KIND == 0) ? __powf(1.f + h.step, h.one_minus_kappa) : 0.f;
  const float floor_p = 1.f / (1.f + h.step);
  const long long n8 = n >> 3;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i8 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i8 < n8; i8 += stride) {
    const long long base = i8 << 3;
    float pv[8], gv[8], mv[8], vv[8], tv[8];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const float4 a = *reinterpret_cast<const float4*>(p + base + q * 4);
      const float4 b = *reinterpret_cast<const float4*>(g + base + q * 4);
      const float4 c = *reinterpret_cast<const float4*>(m + base + q * 4);
      const float4 d = *reinterpret_cast<const float4*>(v + base + q * 4);
      pv[q * 4] = a.x; pv[q * 4 + 1] = a.y; pv[q * 4 + 2] = a.z; pv[q * 4 + 3] = a.w;
      gv[q * 4] = b.x; gv[q * 4 + 1] = b.y; gv[q * 4 + 2] = b.z; gv[q * 4 + 3] = b.w;
      mv[q * 4] = c.x; mv[q * 4 + 1] = c.y; mv[q * 4 + 2] = c.z; mv[q * 4 + 3] = c.w;
      vv[q * 4] = d.x; vv[q * 4 + 1] = d.y; vv[q * 4 + 2] = d.z; vv[q * 4 + 3] = d.w;
      if (KIND == 1 || KIND == 4 || KIND == 5) {
        const float4 e = *reinterpret_cast<const float4*>(tau + base + q * 4);
        tv[q * 4] = e.x; tv[q * 4 + 1] = e.y; tv[q * 4 + 2] = e.z; tv[q * 4 + 3] = e.w;
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gi = gv[k] * gs;
      float pi = pv[k], mi = mv[k], vi = vv[k];
      if (KIND == 0 || KIND == 1) {
        mi = mi + h.alpha * (gi - mi);
        vi = vi * (1.f - h.alpha) + h.alpha * gi * gi;
        const float denom = sqrtf(vi) + h.eps;
        float norm, af, longterm;
        if (KIND == 0) {
          norm = 1.f / denom;
          af = tpow * fabsf(mi) * norm;
          if (h.clipsnr >= 0.f) af = fminf(af, h.clipsnr);
          longterm = sgn(mi) * af + mi * norm;
        } else {
          float ti = tv[k];
          const float ag = fabsf(gi);
          ti = ti + h.alpha * (ag / (ag + denom) - ti);
          tv[k] = ti;
          const float ct = fminf(ti, 0.5f);
          const float reg = fmaxf(ct / (1.f - ct), floor_p);
          const float eff = fmaxf(ti * h.step, 1.f);
          norm = sqrtf(reg) / denom;
          const float mn = fabsf(mi) * norm;
          af = __powf(eff, h.one_minus_kappa) * mn / reg;
          if (h.clipsnr >= 0.f) af = fminf(af, h.clipsnr);
          longterm = sgn(mi) * (reg * af + mn);
        }
        pi += (-h.lr) * gi * norm + (-h.lr) * h.gamma3 * longterm;
        pi *= h.wd_factor;
      } else if (KIND == 4 || KIND == 5) {   // AdEMAMix: the slow EMA lives in the tau buffer (see optim.cu)
        float si = tv[k];
        mi = h.beta1 * mi + (1.f - h.beta1) * gi;
        si = h.beta3 * si + (1.f - h.beta3) * gi;
        vi = h.beta2 * vi + (1.f - h.beta2) * gi * gi;
        tv[k] = si;
        float upd = (mi / h.bc1 + h.alpha * h.gamma3 * si) / (sqrtf(vi) / sqrtf(h.bc2) + h.eps);
        if (KIND == 5) pi *= h.wd_factor;
        else upd += h.wd_coupled * pi;
        pi -= h.lr * upd;
      } else {
        if (KIND == 2) pi *= h.wd_factor;
        mi = h.beta1 * mi + (1.f - h.beta1) * gi;
        vi = h.beta2 * vi + (1.f - h.beta2) * gi * gi;
        pi -= (h.lr / h.bc1) * mi / (sqrtf(vi) / sqrtf(h.bc2) + h.eps);
        if (KIND == 3) pi *= h.wd_factor;
      }
      pv[k] = pi; mv[k] = mi; vv[k] = vi;
    }
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      *reinterpret_cast<float4*>(p + base + q * 4) = make_float4(pv[q * 4], pv[q * 4 + 1], pv[q * 4 + 2], pv[q * 4 + 3]);
      *reinterpret_cast<float4*>(m + base + q * 4) = make_float4(mv[q * 4], mv[q * 4 + 1], mv[q * 4 + 2], mv[q * 4 + 3]);
      *reinterpret_cast<float4*>(v + base + q * 4) = make_float4(vv[q * 4], vv[q * 4 + 1], vv[q * 4 + 2], vv[q * 4 + 3]);
      if (KIND == 1 || KIND == 4 || KIND == 5)
        *reinterpret_cast<float4*>(tau + base + q * 4) = make_float4(tv[q * 4], tv[q * 4 + 1], tv[q * 4 + 2], tv[q * 4 + 3]);
    }
    uint4 packed;
    packed.x = pack_bf16x2(pv[0], pv[1]);
    packed.y = pack_bf16x2(pv[2], pv[3]);
    packed.z = pack_bf16x2(pv[4], pv[5]);
    packed.w = pack_bf16x2(pv[6], pv[7]);
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r) {
      if (r < world)
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(weights.p[r]) + push_off + base) = packed;
    }
  }
}

// Second half of the push-style reduce-scatter (first half: the GEMM epilogue EPI_BF16_PUSH stores every rank's
// partial rows into its slot here): out = resid + sum over slots, fp32 accumulation in slot order, 8 columns per thread.
struct SlotPtrs {
  const __nv_bfloat16* p[8];  // first row of slot s: consecutive slots of one array, or one partial matrix per peer
};
__global__ void __launch_bounds__(256)
sum_slots_bf16_kernel(const SlotPtrs slots, int n_slots, int rows, int N, long long ld_slot,
                      float* __restrict__ out, long long ld_out, const float* __restrict__ resid, long long ld_resid,
                      __nv_bfloat16* __restrict__ out16, long long ld_out16) {
  const int vec_per_row = N >> 3;
  const long long total = (long long)rows * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / vec_per_row);
    const int c = (int)(i - (long long)r * vec_per_row) * 8;
    float acc[8];
    if (resid) {
      const float4 a = *reinterpret_cast<const float4*>(resid + (long long)r * ld_resid + c);
      const float4 b = *reinterpret_cast<const float4*>(resid + (long long)r * ld_resid + c + 4);
      acc[0] = a.x; acc[1] = a.y; acc[2] = a.z; acc[3] = a.w; acc[4] = b.x; acc[5] = b.y; acc[6] = b.z; acc[7] = b.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    }
    uint4 u[8];
#pragma unroll
    for (int sidx = 0; sidx < 8; ++sidx)
      if (sidx < n_slots) u[sidx] = *reinterpret_cast<const uint4*>(slots.p[sidx] + (long long)r * ld_slot + c);
#pragma unroll
    for (int sidx = 0; sidx < 8; ++sidx) {
      if (sidx < n_slots) {
        const float2 p0 = unpack_bf16x2(u[sidx].x), p1 = unpack_bf16x2(u[sidx].y), p2 = unpack_bf16x2(u[sidx].z),
                     p3 = unpack_bf16x2(u[sidx].w);
        acc[0] += p0.x; acc[1] += p0.y; acc[2] += p1.x; acc[3] += p1.y;
        acc[4] += p2.x; acc[5] += p2.y; acc[6] += p3.x; acc[7] += p3.y;
      }
    }
    float* o = out + (long long)r * ld_out + c;
    *reinterpret_cast<float4*>(o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(o + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    if (out16) {
      uint4 w;
      w.x = pack_bf16x2(acc[0], acc[1]);
      w.y = pack_bf16x2(acc[2], acc[3]);
      w.z = pack_bf16x2(acc[4], acc[5]);
      w.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(out16 + (long long)r * ld_out16 + c) = w;
    }
  }
}

// Variable-size all-to-all of rows over peer memory, pull style (expert-parallel dispatch and combine).
// Every rank publishes, in memory its peers can read, a buffer of rows sorted by destination and an int32 table
// [2 * world + world * segs_per_rank]: first row and number of rows of the group it holds for each rank, then the
// row counts of the segments inside the groups (destination rank major: for MoE, one count per routed expert).
// After a barrier over the ranks, rank `me` copies from every peer p the group p holds for it.
// The output holds the peers' segments in rank order; out_counts[p * segs_per_rank + j] receives peer p's counts
// for this rank (what an all-to-all of the count table would deliver).  One warp per row, 16-byte lanes: every
// access over NVLink is a coalesced 512-byte line.  With out == nullptr only the counts are produced.
constexpr int A2A_MAX_SEG = 2048;  // world * segs_per_rank the shared-memory table can hold
struct A2APeers {
  const uint4* buf[MAX_RANKS];
  const int* tab[MAX_RANKS];
};
__global__ void __launch_bounds__(256)
p2p_all_to_all_pull_kernel(A2APeers peers, int me, int world, int segs_per_rank, int vec_per_row,
                           uint4* __restrict__ out, long long max_rows_out, int* __restrict__ out_counts,
                           int* status) {
  __shared__ int s_off[MAX_RANKS], s_cnt[MAX_RANKS], s_start[MAX_RANKS + 1];
  const int n_seg = world * segs_per_rank;
  if (threadIdx.x < world) {
    const int p = threadIdx.x;
    s_off[p] = peers.tab[p][me];
    s_cnt[p] = peers.tab[p][world + me];
  }
  if (blockIdx.x == 0 && out_counts) {
    for (int i = threadIdx.x; i < n_seg; i += blockDim.x) {
      const int p = i / segs_per_rank, j = i - p * segs_per_rank;
      out_counts[i] = peers.tab[p][2 * world + me * segs_per_rank + j];
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int p = 0; p < world; ++p) {
      s_start[p] = acc;
      acc += s_cnt[p];
    }
    s_start[world] = acc;
    if (out && acc > max_rows_out && status) atomicCAS(status, 0, (int)ST_BAD_ARGUMENT);
  }
  __syncthreads();
  if (!out) return;
  long long total = s_start[world];
  if (total > max_rows_out) total = max_rows_out;
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = warp0; row < total; row += n_warps) {
    int p = 0;
#pragma unroll
    for (int q = 1; q < MAX_RANKS; ++q) p += (q < world && row >= s_start[q]) ? 1 : 0;
    const uint4* src = peers.buf[p] + ((long long)s_off[p] + (row - s_start[p])) * vec_per_row;
    uint4* dst = out + row * vec_per_row;
    for (int v = lane; v < vec_per_row; v += 4 * 32) {
      uint4 t[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (v + j * 32 < vec_per_row) t[j] = src[v + j * 32];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (v + j * 32 < vec_per_row) dst[v + j * 32] = t[j];
    }
  }
}

}  // namespace adana

using namespace adana;

static PeerPtrs make_ptrs(const unsigned long long* ptrs, int world) {
  PeerPtrs pp;
  for (int r = 0; r < MAX_RANKS; ++r) pp.p[r] = r < world ? reinterpret_cast<void*>(ptrs[r]) : nullptr;
  return pp;
}

static int grid_for(long long work_items) {
  long long b = (work_items + 255) / 256;
  const long long cap = 148 * 8;
  return (int)(b < 1 ? 1 : (b < cap ? b : cap));
}

extern "C" int adana_p2p_barrier(const unsigned long long* flag_ptrs, int rank, int world, int slot_base,
                                 unsigned int seq, unsigned long long timeout_ns, int* status, void* stream_) {
  if (world < 1 || world > MAX_RANKS) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  p2p_barrier_kernel<<<1, 32, 0, st>>>(make_ptrs(flag_ptrs, world), rank, world, slot_base, seq, timeout_ns, status);
  return (int)cudaGetLastError();
}

extern "C" int adana_p2p_reduce_scatter(const unsigned long long* grad_ptrs, int world, long long shard_off,
                                        long long n, float* out, float* sumsq, void* stream_) {
  if (world < 1 || world > MAX_RANKS || (n & 3) || (shard_off & 3)) return -1;
  if (n == 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  p2p_reduce_scatter_kernel<<<grid_for(n / 4), 256, 0, st>>>(make_ptrs(grad_ptrs, world), world, shard_off, n, out, sumsq);
  return (int)cudaGetLastError();
}

// Largest grid of the gradient collectives that run beside the backward GEMMs.  They have a whole block's backward to
// hide behind (only the last unit's reduction is exposed), so the grid is sized for little interference rather than for
// link speed: on eight GPUs the flagship step took 2179.7 ms with 16 CTAs against 2219.8 ms with 64 (the same step on
// one GPU of such a box: 2171.4 ms), the forward + backward phase alone 2169 against 2209 ms.  A thread keeps one
// 16-byte load per rank in flight, so the cap is given for eight ranks and grows as the ranks get fewer (16 at eight,
// 32 at four, 64 at two, where 64 was measured at 2176.5 ms): the bytes in flight on the links stay the same.
// ADANA_COMM_CTAS sets the cap itself, for every world size.
static int comm_cta_cap(int world) {
  static int forced = -1;
  if (forced < 0) {
    const char* e = getenv("ADANA_COMM_CTAS");
    forced = e ? atoi(e) : 0;
    if (forced < 0) forced = 0;
    if (forced > 148 * 8) forced = 148 * 8;
  }
  if (forced > 0) return forced;
  const int w = world < 1 ? 1 : world;
  const int cap = 16 * MAX_RANKS / w;
  return cap > 128 ? 128 : cap;
}
static int capped_grid(long long work_items, int world) {
  long long b = (work_items + 255) / 256;
  const long long cap = comm_cta_cap(world);
  return (int)(b < 1 ? 1 : (b < cap ? b : cap));
}

extern "C" int adana_p2p_signal(const unsigned long long* flag_ptrs, int rank, int world, int slot,
                                unsigned int seq, void* stream_) {
  if (world < 1 || world > MAX_RANKS || slot < 0) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  p2p_signal_kernel<<<1, 32, 0, st>>>(make_ptrs(flag_ptrs, world), rank, world, slot, seq);
  return (int)cudaGetLastError();
}

// src_ptrs: every rank's copy of the unit (fp32, or bf16 when wire_bf16); my_flags: this rank's flag slots of the
// unit (one per rank; nullptr = do not wait); out fp32 [n]; n and shard_off multiples of 8.
extern "C" int adana_p2p_reduce_scatter_flag(const unsigned long long* src_ptrs, int wire_bf16, const void* my_flags,
                                             unsigned int seq, int world, long long shard_off, long long n,
                                             float* out, float* sumsq, unsigned long long timeout_ns, int* status,
                                             void* stream_) {
  if (world < 1 || world > MAX_RANKS || (n & 7) || (shard_off & 7)) return -1;
  if (n == 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  const int grid = capped_grid(n / 8, world);
  const PeerPtrs src = make_ptrs(src_ptrs, world);
  const uint32_t* fl = reinterpret_cast<const uint32_t*>(my_flags);
  if (wire_bf16)
    p2p_reduce_scatter_flag_kernel<true><<<grid, 256, 0, st>>>(src, fl, seq, world, shard_off, n, out, sumsq, timeout_ns, status);
  else
    p2p_reduce_scatter_flag_kernel<false><<<grid, 256, 0, st>>>(src, fl, seq, world, shard_off, n, out, sumsq, timeout_ns, status);
  return (int)cudaGetLastError();
}

// dst_ptrs: every rank's fp32 gradient buffer of the unit; this rank reduces [slice_off, slice_off + n) and stores it
// on every rank.  May run in place (src == dst, fp32 wire): slices of different ranks are disjoint.
extern "C" int adana_p2p_all_reduce_flag(const unsigned long long* src_ptrs, int wire_bf16,
                                         const unsigned long long* dst_ptrs, const void* my_flags, unsigned int seq,
                                         int world, long long slice_off, long long n, float* sumsq,
                                         unsigned long long timeout_ns, int* status, void* stream_) {
  if (world < 1 || world > MAX_RANKS || (n & 7) || (slice_off & 7)) return -1;
  if (n == 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  const int grid = capped_grid(n / 8, world);
  const PeerPtrs src = make_ptrs(src_ptrs, world), dst = make_ptrs(dst_ptrs, world);
  const uint32_t* fl = reinterpret_cast<const uint32_t*>(my_flags);
  if (wire_bf16)
    p2p_all_reduce_flag_kernel<true><<<grid, 256, 0, st>>>(src, dst, fl, seq, world, slice_off, n, sumsq, timeout_ns, status);
  else
    p2p_all_reduce_flag_kernel<false><<<grid, 256, 0, st>>>(src, dst, fl, seq, world, slice_off, n, sumsq, timeout_ns, status);
  return (int)cudaGetLastError();
}

extern "C" int adana_p2p_publish_f32(const unsigned long long* slot_ptrs, int rank, int world, const float* value,
                                     void* stream_) {
  if (world < 1 || world > MAX_RANKS) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  p2p_publish_f32_kernel<<<1, 32, 0, st>>>(make_ptrs(slot_ptrs, world), rank, world, value);
  return (int)cudaGetLastError();
}

extern "C" int adana_p2p_push_f32(const float* src, const unsigned long long* dst_ptrs, int world, long long dst_off,
                                  long long n, void* stream_) {
  if (world < 1 || world > MAX_RANKS) return -1;
  if (n <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  p2p_push_f32_kernel<<<grid_for(n), 256, 0, st>>>(src, make_ptrs(dst_ptrs, world), world, dst_off, n);
  return (int)cudaGetLastError();
}

extern "C" int adana_clip_coef_multi(const float* partials, int world, float norm_scale, float max_norm, float* out,
                                     void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  clip_coef_multi_kernel<<<1, 1, 0, st>>>(partials, world, norm_scale, max_norm, out);
  return (int)cudaGetLastError();
}

extern "C" int adana_p2p_opt_step_push(float* p, const float* g, float* m, float* v, float* tau,
                                       const unsigned long long* weight_ptrs, int world, long long push_off,
                                       long long n, const AdanaOptHyper* h, const float* clip_coef_ptr,
                                       void* stream_) {
  if (world < 1 || world > MAX_RANKS || (n & 7) || (push_off & 7)) return -1;
  if (n == 0) return 0;
  if ((h->kind == 1 || h->kind == 4 || h->kind == 5) && !tau) return -2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  const int grid = grid_for(n / 8);
  const PeerPtrs w = make_ptrs(weight_ptrs, world);
  switch (h->kind) {
    case 0: p2p_opt_step_push_kernel<0><<<grid, 256, 0, st>>>(p, g, m, v, tau, w, world, push_off, n, *h, clip_coef_ptr); break;
    case 1: p2p_opt_step_push_kernel<1><<<grid, 256, 0, st>>>(p, g, m, v, tau, w, world, push_off, n, *h, clip_coef_ptr); break;
    case 2: p2p_opt_step_push_kernel<2><<<grid, 256, 0, st>>>(p, g, m, v, tau, w, world, push_off, n, *h, clip_coef_ptr); break;
    case 3: p2p_opt_step_push_kernel<3><<<grid, 256, 0, st>>>(p, g, m, v, tau, w, world, push_off, n, *h, clip_coef_ptr); break;
    case 4: p2p_opt_step_push_kernel<4><<<grid, 256, 0, st>>>(p, g, m, v, tau, w, world, push_off, n, *h, clip_coef_ptr); break;
    case 5: p2p_opt_step_push_kernel<5><<<grid, 256, 0, st>>>(p, g, m, v, tau, w, world, push_off, n, *h, clip_coef_ptr); break;
    default: return -3;
  }
  return (int)cudaGetLastError();
}

extern "C" int adana_sum_slots_bf16(const void* slots, int n_slots, int rows, int N, long long ld_slot, float* out,
                                    long long ld_out, const float* resid, long long ld_resid, void* out_bf16,
                                    long long ld_out16, void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (rows <= 0 || N <= 0) return 0;
  if (n_slots < 1 || n_slots > 8 || (N % 8) != 0 || (ld_slot % 8) != 0 || (ld_out % 4) != 0) return -1;
  if ((resid && (ld_resid % 4) != 0) || (out_bf16 && (ld_out16 % 8) != 0)) return -1;
  const long long total = (long long)rows * (N / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  SlotPtrs sp;
  for (int i = 0; i < 8; ++i)
    sp.p[i] = reinterpret_cast<const __nv_bfloat16*>(slots) + (long long)(i < n_slots ? i : 0) * rows * ld_slot;
  sum_slots_bf16_kernel<<<(int)blocks, 256, 0, st>>>(sp, n_slots, rows, N, ld_slot, out, ld_out, resid, ld_resid,
                                                     (__nv_bfloat16*)out_bf16, ld_out16);
  return (int)cudaGetLastError();
}

// Pull-style reduce-scatter of bf16 partial matrices: every rank r holds its partial product P_r [M, N] (pitch ld)
// in memory the others can read; this rank adds rows [first_row, first_row + rows) of all n_ranks partials in fp32,
// in rank order, reading the peers' rows over NVLink with 16-byte coalesced loads.
extern "C" int adana_p2p_reduce_scatter_bf16(const unsigned long long* partial_ptrs, int n_ranks, long long first_row,
                                             int rows, int N, long long ld, float* out, long long ld_out,
                                             const float* resid, long long ld_resid, void* out_bf16,
                                             long long ld_out16, void* stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (rows <= 0 || N <= 0) return 0;
  if (n_ranks < 1 || n_ranks > 8 || (N % 8) != 0 || (ld % 8) != 0 || (ld_out % 4) != 0) return -1;
  if ((resid && (ld_resid % 4) != 0) || (out_bf16 && (ld_out16 % 8) != 0)) return -1;
  SlotPtrs sp;
  for (int i = 0; i < 8; ++i)
    sp.p[i] = reinterpret_cast<const __nv_bfloat16*>(partial_ptrs[i < n_ranks ? i : 0]) + first_row * ld;
  const long long total = (long long)rows * (N / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  sum_slots_bf16_kernel<<<(int)blocks, 256, 0, st>>>(sp, n_ranks, rows, N, ld, out, ld_out, resid, ld_resid,
                                                     (__nv_bfloat16*)out_bf16, ld_out16);
  return (int)cudaGetLastError();
}

// See p2p_all_to_all_pull_kernel.  buf_ptrs[p] / tab_ptrs[p]: peer p's row buffer (row_bytes per row, a multiple of
// 16) and its int32 count table; out may be nullptr (counts only).  Call between two barriers over the ranks.
extern "C" int adana_p2p_all_to_all_pull(const unsigned long long* buf_ptrs, const unsigned long long* tab_ptrs,
                                         int me, int world, int segs_per_rank, long long row_bytes, void* out,
                                         long long max_rows_out, int* out_counts, int* status, void* stream_) {
  if (world < 1 || world > MAX_RANKS || me < 0 || me >= world || segs_per_rank < 1) return -1;
  if (world * segs_per_rank > A2A_MAX_SEG || (row_bytes % 16) != 0 || row_bytes <= 0) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  A2APeers peers;
  for (int p = 0; p < MAX_RANKS; ++p) {
    peers.buf[p] = reinterpret_cast<const uint4*>(buf_ptrs[p < world ? p : 0]);
    peers.tab[p] = reinterpret_cast<const int*>(tab_ptrs[p < world ? p : 0]);
  }
  long long blocks = out ? (max_rows_out + 7) / 8 : 1;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  p2p_all_to_all_pull_kernel<<<(int)blocks, 256, 0, st>>>(peers, me, world, segs_per_rank, (int)(row_bytes / 16),
                                                          reinterpret_cast<uint4*>(out), max_rows_out, out_counts,
                                                          status);
  return (int)cudaGetLastError();
}

ADANA_DBG_BIND(comm)
