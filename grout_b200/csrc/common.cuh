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
#include <stdlib.h>

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

// ---- programmatic dependent launch ------------------------------------------
// A decode step is a chain of short kernels.  Launched with the "programmatic
// stream serialization" attribute, a kernel may become resident while the one
// before it is still draining, do whatever does not depend on that kernel (set
// up addresses, start streaming weights, which no kernel writes), and only then
// wait for it.  pdl_wait() returns once every kernel launched before this one
// has finished and its writes are visible; every kernel that uses it calls it
// before its first read of another kernel's output and before its first global
// write.  pdl_launch_dependents() lets the next kernel in the stream become
// resident; a block calls it once its main loop is over, because blocks of the
// next kernel that arrive earlier only wait while holding registers and shared
// memory that this kernel's own later blocks need (measured: triggering on entry
// made the decode step 25 % slower).  Without the launch attribute both are no-ops.
// The attribute is left off when GROUT_B200_NO_PDL is set in the environment.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
#ifndef GB_PDL_NO_TRIGGER
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}

// A kernel whose whole grid is resident at once (a handful of blocks) loses
// nothing by letting its successor in on entry, and the successor (typically a
// matrix product) can then stream its weights while this kernel runs.
__device__ __forceinline__ bool pdl_small_grid() {
  return gridDim.x * gridDim.y * gridDim.z <= 512;
}
__device__ __forceinline__ void pdl_launch_dependents_if_small() {
  if (pdl_small_grid()) pdl_launch_dependents();
}
__device__ __forceinline__ void pdl_launch_dependents_if_large() {
  if (!pdl_small_grid()) pdl_launch_dependents();
}

static inline bool gb_pdl_enabled() {
  static int on = -1;
  if (on < 0) on = getenv("GROUT_B200_NO_PDL") ? 0 : 1;
  return on == 1;
}

// cluster_x > 1 launches thread-block clusters of that many blocks along x.
template <typename... KArgs, typename... Args>
static inline int gb_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, int cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (gb_pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}

template <typename... KArgs, typename... Args>
static inline int gb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                            cudaStream_t stream, Args... args) {
  return gb_launch_cluster(kernel, grid, block, smem, stream, 1, args...);
}

// Address of row `pos` of kv head `h` of a sequence in a paged cache laid out
// [n_pages, n_kv_heads, page, D]; `table` is the sequence's row of the block table.
__device__ __forceinline__ size_t paged_row(const int* table, int pos, int h, int nkv, int page,
                                            int D) {
  const int pg = table[pos / page];
  return (((size_t)pg * nkv + h) * page + (pos % page)) * (size_t)D;
}
