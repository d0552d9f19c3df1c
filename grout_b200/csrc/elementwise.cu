// Small elementwise kernels: SiLU(gate) * up on the fused gate|up projection,
// and conversions between 32-bit and bfloat16.
#include "common.cuh"

// in [n_rows, 2 I]; with group == 0 the gate is in columns [0, I) and up in
// [I, 2 I); with group g > 0 the columns come in runs of g gates followed by
// their g ups (the layout the decode product's fused epilogue uses).
// out[r, i] = g / (1 + exp(-g)) * u in 32-bit, one rounding at the store
// (the reference's silu_mul_2d_f16, src/kernels.rs:271-296).
template <typename T>
__global__ void silu_mul_kernel(const T* in, T* __restrict__ out, int I, int group) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const size_t r = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= I) return;
  const int gi = group ? (i / group) * 2 * group + (i % group) : i;
  const int ui = group ? gi + group : I + i;
  const float g = to_f32<T>(in[r * 2 * I + gi]);
  const float u = to_f32<T>(in[r * 2 * I + ui]);
  pdl_launch_dependents_if_large();
  out[r * I + i] = from_f32<T>(g / (1.0f + expf(-g)) * u);
}

// bf16, eight outputs per thread in 16-byte pieces: for the plain layout and for
// groups of 8 a thread's gates are 16 contiguous bytes and so are its ups.
__global__ void silu_mul_vec8_kernel(const bf16* in, bf16* __restrict__ out, int I, int group) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const size_t r = blockIdx.y;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;   // which run of 8 outputs
  if (v * 8 >= I) return;
  const bf16* row = in + r * 2 * (size_t)I;
  const bf16* gp = group ? row + (size_t)v * 16 : row + (size_t)v * 8;
  const bf16* up = group ? gp + 8 : row + I + (size_t)v * 8;
  const uint4 g4 = *reinterpret_cast<const uint4*>(gp);
  const uint4 u4 = *reinterpret_cast<const uint4*>(up);
  pdl_launch_dependents_if_large();
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
  const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
  uint4 o4;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float ga = __low2float(g2[k]), gb = __high2float(g2[k]);
    const float ua = __low2float(u2[k]), ub = __high2float(u2[k]);
    o2[k] = __floats2bfloat162_rn(ga / (1.0f + expf(-ga)) * ua, gb / (1.0f + expf(-gb)) * ub);
  }
  *reinterpret_cast<uint4*>(out + r * (size_t)I + (size_t)v * 8) = o4;
}

template <typename T>
static int silu_mul(const void* in, void* out, int n_rows, int I, int group, cudaStream_t s) {
  if (n_rows < 0 || I <= 0 || group < 0 || (group && I % group)) return GB_ERR_BAD_ARG;
  if (n_rows == 0) return 0;
  if (n_rows > 65535) {
    // rows go to grid.y; split very long steps
    for (int r0 = 0; r0 < n_rows; r0 += 65535) {
      const int n = n_rows - r0 < 65535 ? n_rows - r0 : 65535;
      int e = silu_mul<T>((const T*)in + (size_t)r0 * 2 * I, (T*)out + (size_t)r0 * I, n, I, group, s);
      if (e) return e;
    }
    return 0;
  }
  if (sizeof(T) == 2 && I % 8 == 0 && (group == 0 || group == 8) &&
      ((((uintptr_t)in) | ((uintptr_t)out)) & 15) == 0)
    return gb_launch(silu_mul_vec8_kernel, dim3((I / 8 + 127) / 128, n_rows), dim3(128), 0, s,
                     (const bf16*)in, (bf16*)out, I, group);
  return gb_launch(silu_mul_kernel<T>, dim3((I + 255) / 256, n_rows), dim3(256), 0, s,
                   (const T*)in, (T*)out, I, group);
}
GB_EXPORT int gb_silu_mul_f32(const void* in, void* out, int n_rows, int I, int group,
                              cudaStream_t s) {
  return silu_mul<float>(in, out, n_rows, I, group, s);
}
GB_EXPORT int gb_silu_mul_bf16(const void* in, void* out, int n_rows, int I, int group,
                               cudaStream_t s) {
  return silu_mul<bf16>(in, out, n_rows, I, group, s);
}

template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) out[i] = from_f32<TO>(to_f32<TI>(in[i]));
}
template <typename TI, typename TO>
static int cast(const void* in, void* out, long long n, cudaStream_t s) {
  if (n < 0) return GB_ERR_BAD_ARG;
  if (n == 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  cast_kernel<TI, TO><<<(int)blocks, 256, 0, s>>>((const TI*)in, (TO*)out, (size_t)n);
  return gb_status();
}
GB_EXPORT int gb_cast_f32_to_bf16(const void* in, void* out, long long n, cudaStream_t s) {
  return cast<float, bf16>(in, out, n, s);
}
GB_EXPORT int gb_cast_bf16_to_f32(const void* in, void* out, long long n, cudaStream_t s) {
  return cast<bf16, float>(in, out, n, s);
}

// Keeps the stream busy for `ns` nanoseconds (at most a millisecond): one thread
// reads the global timer until the time is up and waits for nothing else.  The
// per-operation profile queues it in front of each timed call so that the host
// has queued the call and its two events before the device reaches them;
// otherwise the time between the events of a short kernel is the host's, not
// the kernel's.
__global__ void delay_kernel(unsigned long long ns) {
  unsigned long long t0, t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
  for (int i = 0; i < (1 << 20); ++i) {          // bounded whatever the timer does
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    if (t - t0 >= ns) break;
    __nanosleep(200);
  }
}
GB_EXPORT int gb_delay_ns(long long ns, cudaStream_t s) {
  if (ns < 0 || ns > 1000000) return GB_ERR_BAD_ARG;
  delay_kernel<<<1, 1, 0, s>>>((unsigned long long)ns);
  return gb_status();
}
