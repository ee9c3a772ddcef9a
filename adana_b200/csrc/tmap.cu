// Host-side tensor-map (TMA descriptor) encoding.  The driver entry point is fetched at run
// time through the CUDA runtime so that the library links without libcuda.
#include "common.cuh"

#include <cudaTypedefs.h>
#include <mutex>
#include <stdio.h>

namespace adana {

static PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
static std::once_flag g_once;

static void load_encode() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) {
    g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  } else {
    fprintf(stderr, "[adana_b200] cuTensorMapEncodeTiled entry point not found (%d)\n", (int)e);
  }
}

int encode_tmap_nd(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                   const uint64_t* strides_elems, const uint32_t* box, int elem_bytes,
                   int swizzle_128) {
  std::call_once(g_once, load_encode);
  if (!g_encode) return -1;
  // The encoder is a driver-API call and needs a context current on THIS thread; a thread that
  // has only ever been handed tensors (PyTorch's autograd worker) may not have one bound yet.
  // cudaSetDevice binds the device's primary context to the calling thread.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -5;
    ctx_bound = true;
  }
  if (rank < 1 || rank > 5) return -2;
  if ((reinterpret_cast<uintptr_t>(base) & 0xF) != 0) return -3;
  cuuint64_t gdim[5];
  cuuint64_t gstride[4];
  cuuint32_t bdim[5];
  cuuint32_t estride[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estride[i] = 1;
    if (i > 0) {
      gstride[i - 1] = strides_elems[i] * (uint64_t)elem_bytes;
      if (gstride[i - 1] % 16 != 0) return -4;
    }
  }
  CUtensorMapDataType dt = elem_bytes == 2   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                             : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = g_encode(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstride, bdim,
                        estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle_128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr,
            "[adana_b200] cuTensorMapEncodeTiled failed: %d (rank %d dims %llu %llu box %u %u)\n",
            (int)r, rank, (unsigned long long)dims[0],
            (unsigned long long)(rank > 1 ? dims[1] : 0), box[0], rank > 1 ? box[1] : 0);
    return (int)r;
  }
  return 0;
}

int encode_tmap_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                   uint64_t ld_elems, uint32_t box_inner, uint32_t box_outer, int elem_bytes) {
  uint64_t dims[2] = {inner, outer};
  uint64_t strides[2] = {1, ld_elems};
  uint32_t box[2] = {box_inner, box_outer};
  return encode_tmap_nd(out, base, 2, dims, strides, box, elem_bytes, 1);
}

}  // namespace adana
