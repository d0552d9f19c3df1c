// gb_gemm_skinny_bf16_noalloc: the decode-time linear layer for callers that
// must not allocate device memory.
//
// This entry point has no counterpart in the reference.  It exists for hosts
// that cannot call cudaMalloc (or any allocating routine, torch's included) at
// the moment they need the product: a serving process that commits all device
// memory to weights and cache at start-up and forbids the allocator afterwards,
// because cudaMalloc stalls every stream of the device and can fail when nothing
// is left; or code that runs as a guest inside another runtime which owns the
// device's memory and offers no allocator to its callbacks.
//
// What it computes is exactly what gb_gemm_skinny_bf16 computes without the
// SiLU epilogue:  y[M, N] = x[M, K] . W[N, K]^T,  bf16 inputs, 32-bit sums,
// M <= 64, K a multiple of 8, x and W 16-byte aligned.  The caller passes the
// inputs and the output; the scratch of the work split (two 32-bit partial
// tiles per block and one arrival counter per tile of weight rows) lives in two file-scope
// `static __device__` arrays inside the library instead of in buffers from an
// allocator:
//
//   GB_NOALLOC_SCRATCH_FLOATS floats (4 MiB) and GB_NOALLOC_MAX_TILES counters
//   (64 KiB).  Every GPU on which the library is loaded holds them until the
//   process exits, whether or not this function is ever called.
//
// A launch whose partial tiles or tile count exceed those sizes is refused with
// GB_ERR_TOO_LARGE (-3) and nothing is launched; use the allocating entry point
// for it.  (On a GPU with 148 SMs every shape with M <= 16 and up to 16384 tiles
// of weight rows fits; M > 16 does not: its tiles are 32 rows by 32 or 64.)
//
// The call itself makes no cudaMalloc, cudaFree or other allocating call.  The
// first call on each device looks up the arrays' device addresses
// (cudaGetSymbolAddress, with that device current) and the SM count; make that
// first call before any stream capture begins on the device.
//
// All calls share the one scratch, and it keeps what the previous call left.
// The counters the launch needs are cleared on `stream` before the kernel; the
// partial tiles need no clearing (each is written before it is read).  Two
// calls that overlap on the GPU (different streams without an ordering between
// them) race on the scratch and give wrong results: order them.
//
// Returns 0, a cudaError_t (positive), or GB_ERR_BAD_ARG (-1) /
// GB_ERR_UNSUPPORTED (-2) / GB_ERR_TOO_LARGE (-3).
#pragma once
#include <cuda_runtime.h>

#define GB_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define GB_NOALLOC_MAX_TILES (1 << 14)
#define GB_NOALLOC_MAX_DEVICES 64
#define GB_ERR_TOO_LARGE (-3)

#ifdef __cplusplus
extern "C" {
#endif

// out_f32: 1 writes float y, 0 writes bf16 y.
int gb_gemm_skinny_bf16_noalloc(const void* x, const void* W, void* y, int M, int N, int K,
                                int out_f32, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
