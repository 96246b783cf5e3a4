// Allocation-free entry point of libkareus_b200.so.
//
// This function has no counterpart in the reference; it exists for callers that cannot allocate
// device memory at the point where they need the kernel: code running while a memory pool is
// frozen, real-time or embedded-style hosts that size all device memory up front, or bindings from
// runtimes that have no allocator to hand us (plain C, another framework's stream callback).
// Every other entry point of the library either takes caller-provided scratch or is wrapped by
// Python code that allocates it through PyTorch.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// RMSNorm backward for bf16 rows:  dx[rows, H], dw[H] (fp32)  from  dy, x [rows, H] (bf16),
// rstd[rows] (fp32, as returned by the forward) and the weight w[H] (bf16).
//
// * Calls no cudaMalloc/cudaFree or any allocating routine.  The per-CTA partial sums of dw go to
//   a fixed array inside the library (148 x 8192 floats, about 4.6 MB, held by every GPU that
//   loads the library until the process exits).
// * Supported: 512 <= H <= 8192, H a multiple of 8, rows >= 1.  Anything else returns 7 and
//   launches nothing.
// * The first call on each device looks up the array's device address (cudaGetSymbolAddress with
//   that device current).  Make that first call outside of any stream capture.
// * All calls on a device share the array and it keeps the previous call's contents; each call
//   overwrites every slot it later reads, so nothing needs clearing, but two calls that overlap on
//   the GPU (different streams) race on it.  Serialise them on one stream or with events.
// Returns 0 on success, 7 for unsupported sizes, 1000+cudaError for a failed address lookup,
// 2000+cudaError for a failed launch.
int kb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const float* rstd, const void* w, void* dx, float* dw,
                           int rows, int H, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
