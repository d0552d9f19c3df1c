// Token embedding: out[t, :] = table[ids[t], :], a pure copy
// (the reference's embedding_batch_f16, src/kernels.rs:693-711).
#include "common.cuh"

template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* ids,
                             T* __restrict__ out, int H, int V) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < V;  // an id outside the table gives a zero row
  const T* src = table + (size_t)(ok ? id : 0) * H;
  T* dst = out + (size_t)t * H;
  const int per16 = 16 / (int)sizeof(T);
  if ((H % per16) == 0 && (((uintptr_t)table | (uintptr_t)out) & 15) == 0) {
    const int4* s4 = reinterpret_cast<const int4*>(src);
    int4* d4 = reinterpret_cast<int4*>(dst);
    const int n = H / per16;
    for (int i = threadIdx.x; i < n; i += blockDim.x) d4[i] = ok ? s4[i] : make_int4(0, 0, 0, 0);
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = ok ? src[i] : from_f32<T>(0.f);
  }
  pdl_launch_dependents_if_large();
}

template <typename T>
static int embed_launch(const void* table, const int* ids, void* out, int n_tokens, int H, int V,
                        cudaStream_t stream) {
  if (n_tokens < 0 || H <= 0 || V <= 0) return GB_ERR_BAD_ARG;
  if (n_tokens == 0) return 0;
  return gb_launch(embed_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, (const T*)table, ids,
                   (T*)out, H, V);
}

GB_EXPORT int gb_embed_f32(const void* table, const int* ids, void* out, int n_tokens, int H, int V,
                           cudaStream_t s) {
  return embed_launch<float>(table, ids, out, n_tokens, H, V, s);
}
GB_EXPORT int gb_embed_bf16(const void* table, const int* ids, void* out, int n_tokens, int H,
                            int V, cudaStream_t s) {
  return embed_launch<bf16>(table, ids, out, n_tokens, H, V, s);
}
