// Entry point for callers that must not allocate device memory.
//
// This function has no counterpart in the reference project: it exists for hosts that embed the kernel
// library where cudaMalloc is off limits -- inside a CUDA-graph capture or another stream-ordered region
// where an allocation would be illegal or would synchronise, in a process that runs under a fixed memory
// budget handed out by an external pool, or in a real-time serving loop that forbids allocator calls.
//
// lmoe_rms_norm_bwd_noalloc computes exactly what lmoe_rms_norm_bwd computes (RMSNorm backward: dx, and dw
// through per-block partial sums), but the partial sums live in a fixed array that is part of the library
// image instead of a caller-provided scratch buffer.
//
//   * The array is LMOE_NOALLOC_MAX_BLOCKS x LMOE_NOALLOC_MAX_N floats (4.6 MiB).  Every GPU that loads the
//     library holds it from load until the process exits.
//   * N (the normalised width) must be <= LMOE_NOALLOC_MAX_N and a multiple of 8 (bf16) or 4 (fp32);
//     otherwise the call returns LMOE_NOALLOC_ERR_SIZE and launches nothing.  rows may be anything from 0 up to
//     2^31 - 1 (the kernels index rows with a 32-bit integer); more is refused with LMOE_NOALLOC_ERR_SIZE too.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress) with that
//     device current.  Make that first call before any stream capture begins.
//   * The function calls no cudaMalloc / cudaFree and no allocating library routine.
//   * All calls share the one array.  Its previous contents are never read before being overwritten (each
//     block writes its whole row of partials before the reduction reads them), so nothing needs clearing;
//     but two calls whose kernels overlap on the GPU (different streams, or different threads on the same
//     device) race on it.  Serialise them on one stream.
//   * inputs and outputs are the caller's: dy, xin [rows, N]; w [N] or null; rstd [rows] fp32;
//     dres [rows, N] or null (added to dx); dx [rows, N]; dw [N] or null.  dtype: 0 = fp32, 1 = bf16.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define LMOE_NOALLOC_MAX_BLOCKS 296
#define LMOE_NOALLOC_MAX_N 4096
#define LMOE_NOALLOC_ERR_SIZE (-100)     /* N too large / not a multiple of the vector width, or rows >= 2^31 */
#define LMOE_NOALLOC_ERR_SETUP (-101)    /* the device address of the scratch array could not be obtained */

#ifdef __cplusplus
extern "C" {
#endif
int lmoe_rms_norm_bwd_noalloc(const void* dy, const void* xin, const void* w, const float* rstd, const void* dres,
                              void* dx, void* dw, int64_t rows, int N, int dtype, cudaStream_t stream);
const char* lmoe_noalloc_strerror(int code);
#ifdef __cplusplus
}
#endif
