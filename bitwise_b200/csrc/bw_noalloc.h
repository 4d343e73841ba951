// Declaration of the one entry point of this library that allocates nothing.
//
// It has no counterpart in the reference (tkran2/bitwise is CPU code and owns all of its
// memory through std::vector): it exists for callers of this GPU library that are not allowed
// to allocate device memory at the moment they need a matrix product.  Think of code that
// runs while a CUDA graph is being captured, inside another framework's stream-ordered
// allocator or memory pool whose bookkeeping an extra cudaMalloc would disturb, in a
// real-time or low-latency loop where the implicit device synchronisation of cudaMalloc /
// cudaFree is not acceptable, or in a process whose memory budget was handed out up front.
// Such callers pass inputs and outputs that they already own; everything else the product
// needs lives in a fixed array inside the library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest scratch the entry point can serve, in floats.  A product that the library splits
// along k (at most 128 rows, more than one chunk of 512 along k, too few output columns to
// occupy the GPU otherwise) uses ceil(k / 512) * m * n floats of it; other products use none.
// bw_bf16_linear_noalloc_scratch_floats tells for a shape.  16 MiB of device memory per GPU
// that loads the library, held until the process exits.
#define BW_NOALLOC_MAX_SCRATCH_FLOATS (4 * 1024 * 1024)

// Floats of scratch that a product of this shape uses (0 when it is not split along k); the
// entry point refuses a product that needs more than BW_NOALLOC_MAX_SCRATCH_FLOATS.
long long bw_bf16_linear_noalloc_scratch_floats(int m, int n, int k);

// y[m][n] = sum_k x[m][k] * w[n][k] (+ residual[m][n]) in bfloat16 with float32 accumulation,
// the same kernels and the same summation order as bw_bf16_linear, so the same bits.
//   x, w      bfloat16, row-major, rows starting on 16 bytes (k a multiple of 8)
//   y         bfloat16 or float32 (y_is_f32), may alias residual
//   residual  float32 or null (then y_is_f32 may be 0 or 1)
// Returns 0 on success; a negative value with bw_last_error() set when the shape is not
// supported or needs more scratch than BW_NOALLOC_MAX_SCRATCH_FLOATS; a CUDA error code
// otherwise.  It calls neither cudaMalloc nor cudaFree nor any routine that allocates.
//
// The first call on a device, with that device current, does the set-up for that device: it
// looks up the device address of the library's scratch array (cudaGetSymbolAddress) and raises
// the shared-memory limit of every kernel variant that any later call may choose, whatever
// its shape.  Make that first call outside any stream capture.  All calls share the one scratch array: two calls whose
// kernels may run at the same time (different streams, or graphs replayed concurrently) race
// on it and give wrong results; calls on one stream are safe.
int bw_bf16_linear_noalloc(const __nv_bfloat16* x, const __nv_bfloat16* w, void* y, int y_is_f32,
                           const float* residual, int m, int n, int k, cudaStream_t stream);

// 1 (once) when a kernel launched by bw_bf16_linear_noalloc gave up a bounded wait since the
// last call of this function, else 0.
int bw_bf16_linear_noalloc_failed(void);

#ifdef __cplusplus
}
#endif
