// Norm backward with a built-in scratch buffer: one C entry point that allocates nothing.
//
// This entry point has no counterpart in the reference; it exists for callers of the kernel library
// that cannot hand in a scratch buffer of their own.
//
// Who needs it.  `adana_norm_bwd` leaves the weight gradient as one partial row per CTA in a caller-provided
// fp32 buffer and `adana_colsum_f32` folds those rows.  The Python wrapper takes that buffer from PyTorch's
// caching allocator.  A caller without such an allocator has nowhere to get it from at step time: a plain
// C or C++ host loop that links the library directly; a runtime that hands out all device memory once at
// start-up and must not call cudaMalloc afterwards (cudaMalloc synchronises the whole device and, late in
// a long run on a nearly full GPU, can fail); a thread that may not take the allocator's lock.  For them
// the partial rows live in a file-scope `__device__` array inside the library, so the call needs no
// memory beyond its arguments.
//
// Limits.  The scratch holds ADANA_NORM_STATIC_MAX_PARTIAL_ROWS x ADANA_NORM_STATIC_MAX_COLS floats
// (444 x 4096 x 4 B = 6.9 MiB per device, reserved when the library's module is loaded).  `cols` above
// ADANA_NORM_STATIC_MAX_COLS, or not a multiple of 4, is rejected with ADANA_NORM_STATIC_E_COLS before
// anything is launched, with a one-line message on stderr; `rows` is unlimited (the grid is capped at the
// number of partial rows and strides over the rows).
//
// Set-up.  The first call on each device looks the array's address up with cudaGetSymbolAddress (which may
// load the module) and caches it; every later call on that device only launches the two kernels.  Make
// that first call during start-up, outside any stream capture and before timing.
//
// Device.  The address is looked up for the CURRENT device (cudaGetDevice), not for the device that `stream`
// belongs to: make the stream's device current before the call, as for any kernel launch.  `mean` may be null
// for RMSNorm (kind 1), which never reads it.  With `rows` <= 0 nothing is launched; `dw` is then set to zero
// (a memset on `stream`) unless `accumulate_dw` is set.
//
// Initial state.  Nothing has to start at zero: every CTA overwrites its whole partial row before the
// fold reads it.  `dw` is overwritten unless `accumulate_dw` is set, `dx` is overwritten unless
// `accumulate_dx` is set; in the accumulate modes the caller owns the initial contents.
//
// Concurrency.  There is ONE scratch array per device.  Calls on the same device are safe back to back
// on one stream.  Calls that can overlap (different streams without an ordering between them, or several
// host threads launching at once) race on the scratch and give wrong weight gradients; order them
// with events or use `adana_norm_bwd` with separate buffers instead.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define ADANA_NORM_STATIC_MAX_PARTIAL_ROWS 444
#define ADANA_NORM_STATIC_MAX_COLS 4096

#define ADANA_NORM_STATIC_E_COLS (-21)    // cols > ADANA_NORM_STATIC_MAX_COLS or cols % 4 != 0
#define ADANA_NORM_STATIC_E_ARG (-22)     // a required pointer is null
#define ADANA_NORM_STATIC_E_SYMBOL (-23)  // the scratch address could not be obtained (CUDA error on stderr)

// dx (fp32 [rows, cols]) and dw (fp32 [cols]) of LayerNorm (kind 0, weight only) or RMSNorm (kind 1).
// dy / x may be bf16 or fp32 as in adana_norm_bwd; dx_bf16 (optional) receives a bf16 copy of the final dx.
// Returns 0, one of the codes above, a negative code of adana_norm_bwd, or a cudaError_t (> 0).
int adana_norm_bwd_static_scratch(const void* dy, int dy_is_bf16, const void* x, int x_is_bf16,
                                  const float* w, const float* mean, const float* rstd, float* dx,
                                  int accumulate_dx, float* dw, int accumulate_dw, int rows, int cols,
                                  int kind, void* dx_bf16, void* stream);

#ifdef __cplusplus
}
#endif
