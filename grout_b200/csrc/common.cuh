// Shared device helpers for the sm_100a kernels of this library.
//
// Every exported function is plain C (`extern "C"`), takes raw device pointers,
// sizes and the CUDA stream to launch on, allocates nothing, and returns 0 or a
// cudaError_t value (positive) or one of the GB_ERR_* codes (negative) when it
// refuses its arguments.  The Python side turns a non-zero return into an
// exception, so a refused size is never a wrong result.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define GB_EXPORT extern "C" __attribute__((visibility("default")))

#define GB_ERR_BAD_ARG (-1)      // a size or pointer the kernel does not take
#define GB_ERR_UNSUPPORTED (-2)  // a combination that has no kernel

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum with a fixed tree, so the result depends on the block size
// only.  `scratch` holds 32 floats.  Every thread gets the sum.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : 0.f;
  r = warp_sum(r);
  return r;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

static inline int gb_status() { return (int)cudaGetLastError(); }

// Address of row `pos` of kv head `h` of a sequence in a paged cache laid out
// [n_pages, n_kv_heads, page, D]; `table` is the sequence's row of the block table.
__device__ __forceinline__ size_t paged_row(const int* table, int pos, int h, int nkv, int page,
                                            int D) {
  const int pg = table[pos / page];
  return (((size_t)pg * nkv + h) * page + (pos % page)) * (size_t)D;
}
