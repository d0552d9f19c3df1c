// RMSNorm with the residual sum folded in.
//
//   v   = res_in[s, :] + delta[s, :]        (either may be absent; 32-bit sum)
//   res_out[r, :] = v                       (32-bit residual stream, optional)
//   y[r, :] = v / sqrt(mean(v^2) + eps) * w
//
// s = rows[r] when a row list is given (gather before the final norm), else r.
// The reference's rms_norm_f16 (src/kernels.rs:304-343) and add_rms_norm_f16
// (src/kernels.rs:3013-3074) keep the sum in f32 only inside the kernel and
// store a 16-bit residual; here the residual stream itself stays 32-bit.
// In 32-bit the kernel, and with it the reduction tree, is chosen by N only, so
// a row's result does not depend on the batch it is in; in bfloat16 few rows of a
// wide model take a cluster of blocks per row (another order of sums, which
// bfloat16's rounding of y hides).
#include <cooperative_groups.h>

#include <type_traits>

#include "common.cuh"

namespace cg = cooperative_groups;

// `parts`: instead of (or beside) delta, n_parts 32-bit partial sums [n_parts]
// [rows_total, N], part_stride floats apart, added in order: the split-K product
// of the projection before this norm leaves its reduction to this kernel.
template <typename T, typename WT>
__global__ void add_rmsnorm_kernel(const float* res_in, const T* delta, const float* parts,
                                   int n_parts, long long part_stride,
                                   const int* __restrict__ rows, const WT* __restrict__ w,
                                   float eps, float* res_out, T* __restrict__ y, int N) {
  __shared__ float scratch[32];
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int r = blockIdx.x;
  const size_t s = rows ? (size_t)rows[r] : (size_t)r;
  const float* rin = res_in ? res_in + s * N : nullptr;
  const T* din = delta ? delta + s * N : nullptr;
  float* rout = res_out ? res_out + (size_t)r * N : nullptr;
  const float* pin = parts ? parts + s * N : nullptr;
  auto value = [&](int i) {
    float d = din ? to_f32<T>(din[i]) : 0.f;
    for (int k = 0; k < n_parts; ++k) d += pin[(size_t)k * part_stride + i];
    return (rin ? rin[i] : 0.f) + d;
  };
  float ss = 0.f;
  for (int i = threadIdx.x; i < N; i += blockDim.x) {
    float v = value(i);
    if (rout) rout[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  pdl_launch_dependents_if_large();
  const float inv = 1.0f / sqrtf(ss / (float)N + eps);
  T* yo = y + (size_t)r * N;
  for (int i = threadIdx.x; i < N; i += blockDim.x) {
    // the same thread wrote rout[i] above, so it reads its own store here
    float v = rout ? rout[i] : value(i);
    yo[i] = from_f32<T>(v * inv * to_f32<WT>(w[i]));
  }
}

// The same operation for widths that are a multiple of 4 and at most 16384:
// every thread keeps its (up to 16) values in registers between the sum of
// squares and the scaling, and all traffic is in 8- or 16-byte pieces.
#define NV_MAX 4
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Vec4<bf16> {
  static __device__ __forceinline__ void load(const bf16* p, float (&v)[4]) {
    const uint2 x = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&x.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&x.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
  }
  static __device__ __forceinline__ void store(bf16* p, const float (&v)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 x;
    x.x = *reinterpret_cast<uint32_t*>(&a);
    x.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = x;
  }
};

template <typename T, typename WT>
__global__ void add_rmsnorm_vec_kernel(const float* res_in, const T* delta, const float* parts,
                                       int n_parts, long long part_stride,
                                       const int* __restrict__ rows, const WT* __restrict__ w,
                                       float eps, float* res_out, T* __restrict__ y, int N) {
  __shared__ float scratch[32];
  pdl_launch_dependents_if_small();
  // the weight vector is no kernel's output: fetch it while the producer drains
  float wv[NV_MAX][4];
#pragma unroll
  for (int j = 0; j < NV_MAX; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
    if (i < N) Vec4<WT>::load(w + i, wv[j]);
  }
  pdl_wait();
  const int r = blockIdx.x;
  const size_t s = rows ? (size_t)rows[r] : (size_t)r;
  const float* rin = res_in ? res_in + s * N : nullptr;
  const T* din = delta ? delta + s * N : nullptr;
  float* rout = res_out ? res_out + (size_t)r * N : nullptr;
  const float* pin = parts ? parts + s * N : nullptr;
  float v[NV_MAX][4];
  float ss = 0.f;
  // all of a thread's loads first, then the sums: the memory system sees every
  // request of the row at once
  float av[NV_MAX][4], dv[NV_MAX][4];
#pragma unroll
  for (int j = 0; j < NV_MAX; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
#pragma unroll
    for (int e = 0; e < 4; ++e) av[j][e] = dv[j][e] = 0.f;
    if (i < N) {
      if (rin) Vec4<float>::load(rin + i, av[j]);
      if (din) Vec4<T>::load(din + i, dv[j]);
    }
  }
#pragma unroll
  for (int j = 0; j < NV_MAX; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
    if (i < N) {
      for (int k0 = 0; k0 < n_parts; k0 += 4) {   // four at once, added in order
        float pk[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int k = k0 + u < n_parts ? k0 + u : n_parts - 1;
          Vec4<float>::load(pin + (size_t)k * part_stride + i, pk[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (k0 + u < n_parts) {
#pragma unroll
            for (int e = 0; e < 4; ++e) dv[j][e] += pk[u][e];
          }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        v[j][e] = av[j][e] + dv[j][e];
        ss += v[j][e] * v[j][e];
      }
      if (rout) Vec4<float>::store(rout + i, v[j]);
    }
  }
  ss = block_sum(ss, scratch);
  pdl_launch_dependents_if_large();
  const float inv = 1.0f / sqrtf(ss / (float)N + eps);
  T* yo = y + (size_t)r * N;
#pragma unroll
  for (int j = 0; j < NV_MAX; ++j) {
    const int i = (threadIdx.x + j * blockDim.x) * 4;
    if (i < N) {
      float o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = v[j][e] * inv * wv[j][e];
      Vec4<T>::store(yo + i, o);
    }
  }
}

// A handful of rows (a decode step) would keep a handful of SMs busy.  Here a
// cluster of NC_CLUSTER blocks shares a row: each block owns a quarter of the
// columns, the sums of squares meet through distributed shared memory (added in
// rank order, so the result is a fixed sum), and every block scales its columns.
// The cluster barrier is the hardware's; no block spins on memory.
#ifndef NC_CLUSTER
#define NC_CLUSTER 4
#endif
template <typename T, typename WT>
__global__ void add_rmsnorm_cluster_kernel(const float* res_in, const T* delta, const float* parts, int n_parts,
                           long long part_stride, const int* __restrict__ rows,
                           const WT* __restrict__ w, float eps, float* res_out,
                           T* __restrict__ y, int N) {
  __shared__ float scratch[32];
  __shared__ float ss_all[NC_CLUSTER];
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  pdl_launch_dependents_if_small();
  const int cols = N / NC_CLUSTER;              // a multiple of 4
  const int c0 = rank * cols;
  const int i = c0 + threadIdx.x * 4;           // this thread's four columns
  const bool active = threadIdx.x * 4 < cols;
  float wv[4] = {0.f, 0.f, 0.f, 0.f};
  if (active) Vec4<WT>::load(w + i, wv);        // no kernel's output: before the wait
  pdl_wait();
  const int r = blockIdx.x / NC_CLUSTER;
  const size_t s = rows ? (size_t)rows[r] : (size_t)r;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  float ss = 0.f;
  if (active) {
    float a[4] = {0.f, 0.f, 0.f, 0.f}, d[4] = {0.f, 0.f, 0.f, 0.f};
    if (res_in) Vec4<float>::load(res_in + s * N + i, a);
    if (delta) Vec4<T>::load(delta + s * N + i, d);
    // eight partials are requested at once and then added in order: one at a time, each
    // load would wait for the one before it to have been added (a round trip to L2 each;
    // a product is split at most eight ways, so this is one trip)
    for (int k0 = 0; k0 < n_parts; k0 += 8) {
      float pk[8][4];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int k = k0 + u < n_parts ? k0 + u : n_parts - 1;
        Vec4<float>::load(parts + (size_t)k * part_stride + s * N + i, pk[u]);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (k0 + u < n_parts) {
#pragma unroll
          for (int e = 0; e < 4; ++e) d[e] += pk[u][e];
        }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      v[e] = a[e] + d[e];
      ss += v[e] * v[e];
    }
    if (res_out) Vec4<float>::store(res_out + (size_t)r * N + i, v);
  }
  ss = block_sum(ss, scratch);
  // every block puts its sum into every block's table (thread k writes to block k), so
  // that one cluster barrier is enough: after it each block reads its own shared memory
  // only, and nobody is read from after it has left
  if (threadIdx.x < NC_CLUSTER) cluster.map_shared_rank(ss_all, threadIdx.x)[rank] = ss;
  cluster.sync();
  float total = 0.f;
#pragma unroll
  for (int k = 0; k < NC_CLUSTER; ++k) total += ss_all[k];
  const float inv = 1.0f / sqrtf(total / (float)N + eps);
  if (active) {
    float o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = v[e] * inv * wv[e];
    Vec4<T>::store(y + (size_t)r * N + i, o);
  }
}

static int norm_threads(int N) {
  int t = (N + 3) / 4;
  t = ((t + 31) / 32) * 32;
  if (t < 32) t = 32;
  if (t > 1024) t = 1024;
  return t;
}

template <typename T, typename WT>
static int launch(const float* res_in, const void* delta, const float* parts, int n_parts,
                  long long part_stride, const int* rows, const void* w, float eps,
                  float* res_out, void* y, int n_rows, int N, cudaStream_t stream) {
  if (n_rows < 0 || N <= 0 || !w || !y || (!res_in && !delta && !parts)) return GB_ERR_BAD_ARG;
  if ((parts != nullptr) != (n_parts > 0) || n_parts < 0) return GB_ERR_BAD_ARG;
  // in place is allowed only without a row list (each block then owns its row)
  if (rows && res_out && res_out == res_in) return GB_ERR_BAD_ARG;
  if (n_rows == 0) return 0;
  const bool aligned = ((((uintptr_t)res_in) | ((uintptr_t)delta) | ((uintptr_t)w) |
                         ((uintptr_t)res_out) | ((uintptr_t)y) | ((uintptr_t)parts) |
                         ((uintptr_t)(part_stride * 4))) & 15) == 0;
  // The cluster kernel is chosen by the number of rows and sums in another order
  // than the kernels below.  The 32-bit path never takes it: there the order of
  // a row's sums may depend on the width alone, so that a token's result is the
  // same in a step of one row and in a step of thousands.
  constexpr bool by_rows_too = !std::is_same<T, float>::value;
#ifndef NC_MAX_ROWS
#define NC_MAX_ROWS 64
#endif
  if (by_rows_too && aligned && n_rows <= NC_MAX_ROWS && N >= 1024 && N % (4 * NC_CLUSTER) == 0 &&
      N / NC_CLUSTER <= 4096) {
    int threads = ((N / NC_CLUSTER / 4 + 31) / 32) * 32;
    return gb_launch_cluster(add_rmsnorm_cluster_kernel<T, WT>, dim3(n_rows * NC_CLUSTER),
                             dim3(threads), 0, stream, NC_CLUSTER, res_in, (const T*)delta, parts,
                             n_parts, part_stride, rows, (const WT*)w, eps, res_out, (T*)y, N);
  }
  if (N % 4 == 0 && N <= 4 * 1024 * NV_MAX && aligned) {
    int threads = (N / 4 + NV_MAX - 1) / NV_MAX;      // vectors per thread <= NV_MAX
    threads = ((threads + 31) / 32) * 32;
    if (threads < 64) threads = 64;
    if (threads > 1024) threads = 1024;
    return gb_launch(add_rmsnorm_vec_kernel<T, WT>, dim3(n_rows), dim3(threads), 0, stream, res_in,
                     (const T*)delta, parts, n_parts, part_stride, rows, (const WT*)w, eps, res_out,
                     (T*)y, N);
  }
  return gb_launch(add_rmsnorm_kernel<T, WT>, dim3(n_rows), dim3(norm_threads(N)), 0, stream, res_in,
                   (const T*)delta, parts, n_parts, part_stride, rows, (const WT*)w, eps, res_out,
                   (T*)y, N);
}

// w_is_f32: the weight vector is stored in 32-bit although the activations are bf16.
GB_EXPORT int gb_add_rmsnorm_f32(const float* res_in, const void* delta, const float* parts,
                                 int n_parts, long long part_stride, const int* rows,
                                 const void* w, int w_is_f32, float eps, float* res_out, void* y,
                                 int n_rows, int N, cudaStream_t s) {
  if (!w_is_f32) return GB_ERR_UNSUPPORTED;
  return launch<float, float>(res_in, delta, parts, n_parts, part_stride, rows, w, eps, res_out, y,
                              n_rows, N, s);
}
GB_EXPORT int gb_add_rmsnorm_bf16(const float* res_in, const void* delta, const float* parts,
                                  int n_parts, long long part_stride, const int* rows,
                                  const void* w, int w_is_f32, float eps, float* res_out, void* y,
                                  int n_rows, int N, cudaStream_t s) {
  if (w_is_f32)
    return launch<bf16, float>(res_in, delta, parts, n_parts, part_stride, rows, w, eps, res_out, y,
                               n_rows, N, s);
  return launch<bf16, bf16>(res_in, delta, parts, n_parts, part_stride, rows, w, eps, res_out, y,
                            n_rows, N, s);
}
