// See norm_static_scratch.h: norm backward whose per-CTA weight-gradient rows live in a static device array.
#include <cuda_runtime.h>

#include <cstdio>

#include "api.h"
#include "norm_static_scratch.h"

namespace {

// One partial row per CTA of the backward kernel; overwritten in full by every call (no zeroing needed).
static __device__ __align__(256) float g_dw_partial_scratch[(size_t)ADANA_NORM_STATIC_MAX_PARTIAL_ROWS *
                                                            ADANA_NORM_STATIC_MAX_COLS];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {};  // device address of the array above, per device, filled on first use

int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    std::fprintf(stderr, "adana_norm_bwd_static_scratch: cudaGetDevice failed or device %d out of range: %s\n", dev,
                 cudaGetErrorString(e));
    return ADANA_NORM_STATIC_E_SYMBOL;
  }
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_dw_partial_scratch);
    if (e != cudaSuccess || p == nullptr) {
      std::fprintf(stderr, "adana_norm_bwd_static_scratch: cudaGetSymbolAddress failed on device %d: %s\n", dev,
                   cudaGetErrorString(e));
      return ADANA_NORM_STATIC_E_SYMBOL;
    }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace

extern "C" int adana_norm_bwd_static_scratch(const void* dy, int dy_is_bf16, const void* x, int x_is_bf16,
                                             const float* w, const float* mean, const float* rstd, float* dx,
                                             int accumulate_dx, float* dw, int accumulate_dw, int rows, int cols,
                                             int kind, void* dx_bf16, void* stream) {
  if (cols <= 0 || (cols & 3) || cols > ADANA_NORM_STATIC_MAX_COLS) {
    std::fprintf(stderr,
                 "adana_norm_bwd_static_scratch: cols=%d rejected: must be a multiple of 4 and at most %d "
                 "(the built-in scratch holds %d x %d floats); use adana_norm_bwd with your own buffer\n",
                 cols, ADANA_NORM_STATIC_MAX_COLS, ADANA_NORM_STATIC_MAX_PARTIAL_ROWS, ADANA_NORM_STATIC_MAX_COLS);
    return ADANA_NORM_STATIC_E_COLS;
  }
  // RMSNorm (kind 1) never reads `mean`, so its callers need not invent a buffer for it.
  if (!dy || !x || !w || (kind == 0 && !mean) || !rstd || !dx || !dw) {
    std::fprintf(stderr, "adana_norm_bwd_static_scratch: null pointer among dy/x/w/mean/rstd/dx/dw\n");
    return ADANA_NORM_STATIC_E_ARG;
  }
  if (rows <= 0) {
    // no rows: the weight gradient of an empty batch is zero (an accumulating call leaves dw as it is)
    if (!accumulate_dw) {
      cudaError_t e = cudaMemsetAsync(dw, 0, sizeof(float) * (size_t)cols, reinterpret_cast<cudaStream_t>(stream));
      if (e != cudaSuccess) return (int)e;
    }
    return 0;
  }
  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  const int parts = rows < ADANA_NORM_STATIC_MAX_PARTIAL_ROWS ? rows : ADANA_NORM_STATIC_MAX_PARTIAL_ROWS;
  rc = adana_norm_bwd(dy, dy_is_bf16, x, x_is_bf16, w, mean, rstd, dx, accumulate_dx, scratch, parts, rows, cols,
                      kind, dx_bf16, stream);
  if (rc) return rc;
  return adana_colsum_f32(scratch, parts, cols, dw, accumulate_dw, stream);
}
