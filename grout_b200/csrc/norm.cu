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
// The reduction tree depends on N only, so a row's result does not depend on
// the batch it is in.
#include "common.cuh"

template <typename T, typename WT>
__global__ void add_rmsnorm_kernel(const float* res_in, const T* __restrict__ delta,
                                   const int* __restrict__ rows, const WT* __restrict__ w,
                                   float eps, float* res_out, T* __restrict__ y, int N) {
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const size_t s = rows ? (size_t)rows[r] : (size_t)r;
  const float* rin = res_in ? res_in + s * N : nullptr;
  const T* din = delta ? delta + s * N : nullptr;
  float* rout = res_out ? res_out + (size_t)r * N : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < N; i += blockDim.x) {
    float v = (rin ? rin[i] : 0.f) + (din ? to_f32<T>(din[i]) : 0.f);
    if (rout) rout[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)N + eps);
  T* yo = y + (size_t)r * N;
  for (int i = threadIdx.x; i < N; i += blockDim.x) {
    // the same thread wrote rout[i] above, so it reads its own store here
    float v = rout ? rout[i] : ((rin ? rin[i] : 0.f) + (din ? to_f32<T>(din[i]) : 0.f));
    yo[i] = from_f32<T>(v * inv * to_f32<WT>(w[i]));
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
static int launch(const float* res_in, const void* delta, const int* rows, const void* w, float eps,
                  float* res_out, void* y, int n_rows, int N, cudaStream_t stream) {
  if (n_rows < 0 || N <= 0 || !w || !y || (!res_in && !delta)) return GB_ERR_BAD_ARG;
  // in place is allowed only without a row list (each block then owns its row)
  if (rows && res_out && res_out == res_in) return GB_ERR_BAD_ARG;
  if (n_rows == 0) return 0;
  add_rmsnorm_kernel<T, WT><<<n_rows, norm_threads(N), 0, stream>>>(
      res_in, (const T*)delta, rows, (const WT*)w, eps, res_out, (T*)y, N);
  return gb_status();
}

// w_is_f32: the weight vector is stored in 32-bit although the activations are bf16.
GB_EXPORT int gb_add_rmsnorm_f32(const float* res_in, const void* delta, const int* rows,
                                 const void* w, int w_is_f32, float eps, float* res_out, void* y,
                                 int n_rows, int N, cudaStream_t s) {
  if (!w_is_f32) return GB_ERR_UNSUPPORTED;
  return launch<float, float>(res_in, delta, rows, w, eps, res_out, y, n_rows, N, s);
}
GB_EXPORT int gb_add_rmsnorm_bf16(const float* res_in, const void* delta, const int* rows,
                                  const void* w, int w_is_f32, float eps, float* res_out, void* y,
                                  int n_rows, int N, cudaStream_t s) {
  if (w_is_f32) return launch<bf16, float>(res_in, delta, rows, w, eps, res_out, y, n_rows, N, s);
  return launch<bf16, bf16>(res_in, delta, rows, w, eps, res_out, y, n_rows, N, s);
}
