// Plain attention over the paged cache, one block per (token, query head):
// the same code for whole prompts and for single decoded tokens, with all
// arithmetic in 32-bit.  It is the attention of the 32-bit path and the
// fallback of the bf16 path for shapes the fast kernels refuse.
//
// Keys lo..pos of the token's sequence are visited in chunks of ATT_THREADS in
// increasing order with an online softmax (running max m, running sum l), so a
// token's result depends only on its own keys: not on the step it is part of,
// the other sequences of the batch, or where its pages lie.
// Scores are q.k * scale; key j is visible when j <= pos and, with a window W,
// when j > pos - W (the reference masks with -1e30 instead of skipping,
// src/kernels.rs:1190-1191, 1256; same result).
#include "common.cuh"

#define ATT_THREADS 128
#define ATT_MAX_ACC 4  // head_dim <= ATT_THREADS * ATT_MAX_ACC

template <typename T>
__global__ void attn_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pages,
                                    const T* __restrict__ v_pages,
                                    const int* __restrict__ block_table, int max_pages,
                                    const int* __restrict__ token_seq,
                                    const int* __restrict__ token_pos,
                                    const int* __restrict__ slots, T* __restrict__ out, int nq,
                                    int nkv, int D, int page, float scale, int window) {
  extern __shared__ float sm[];
  __shared__ float scratch[32];
  float* q_s = sm;       // [D]
  float* p_s = sm + D;   // [ATT_THREADS]
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int slot = slots[token_seq[t]];
  T* o = out + ((size_t)t * nq + h) * D;
  if (slot < 0) {  // padding row
    for (int d = tid; d < D; d += ATT_THREADS) o[d] = from_f32<T>(0.f);
    return;
  }
  const int pos = token_pos[t];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int kvh = h / (nq / nkv);
  const int* table = block_table + (size_t)slot * max_pages;
  const T* qr = q + ((size_t)t * nq + h) * D;
  for (int d = tid; d < D; d += ATT_THREADS) q_s[d] = to_f32<T>(qr[d]);
  __syncthreads();

  float m = -INFINITY, l = 0.f;
  float acc[ATT_MAX_ACC];
#pragma unroll
  for (int i = 0; i < ATT_MAX_ACC; ++i) acc[i] = 0.f;

  for (int c = lo; c <= pos; c += ATT_THREADS) {
    const int j = c + tid;
    const bool valid = j <= pos;
    float s = -INFINITY;
    if (valid) {
      const T* kr = k_pages + paged_row(table, j, kvh, nkv, page, D);
      float a = 0.f;
      for (int d = 0; d < D; ++d) a = fmaf(q_s[d], to_f32<T>(kr[d]), a);
      s = a * scale;
    }
    const float cmax = block_max(s, scratch);  // key c is always valid, so finite
    const float m_new = fmaxf(m, cmax);
    const float p = valid ? expf(s - m_new) : 0.f;
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    p_s[tid] = p;
    const float csum = block_sum(p, scratch);  // its barriers also publish p_s
    l = l * corr + csum;
    const int n = min(ATT_THREADS, pos - c + 1);
#pragma unroll
    for (int i = 0; i < ATT_MAX_ACC; ++i) acc[i] *= corr;
    for (int jj = 0; jj < n; ++jj) {
      const T* vr = v_pages + paged_row(table, c + jj, kvh, nkv, page, D);
      const float pj = p_s[jj];
#pragma unroll
      for (int i = 0; i < ATT_MAX_ACC; ++i) {
        const int d = tid + i * ATT_THREADS;
        if (d < D) acc[i] = fmaf(pj, to_f32<T>(vr[d]), acc[i]);
      }
    }
    m = m_new;
    __syncthreads();  // p_s is rewritten by the next chunk
  }
  const float inv_l = 1.0f / l;
#pragma unroll
  for (int i = 0; i < ATT_MAX_ACC; ++i) {
    const int d = tid + i * ATT_THREADS;
    if (d < D) o[d] = from_f32<T>(acc[i] * inv_l);
  }
}

template <typename T>
static int launch(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                  int max_pages, const int* token_seq, const int* token_pos, const int* slots,
                  void* out, int n_tokens, int nq, int nkv, int D, int page, float scale,
                  int window, cudaStream_t stream) {
  if (n_tokens < 0 || nq <= 0 || nkv <= 0 || nq % nkv || D <= 0 || page <= 0 || max_pages <= 0)
    return GB_ERR_BAD_ARG;
  if (D > ATT_THREADS * ATT_MAX_ACC) return GB_ERR_UNSUPPORTED;
  if (n_tokens == 0) return 0;
  const size_t smem = (size_t)(D + ATT_THREADS) * sizeof(float);
  attn_generic_kernel<T><<<dim3(n_tokens, nq), ATT_THREADS, smem, stream>>>(
      (const T*)q, (const T*)k_pages, (const T*)v_pages, block_table, max_pages, token_seq,
      token_pos, slots, (T*)out, nq, nkv, D, page, scale, window);
  return gb_status();
}

GB_EXPORT int gb_attn_generic_f32(const void* q, const void* k_pages, const void* v_pages,
                                  const int* block_table, int max_pages, const int* token_seq,
                                  const int* token_pos, const int* slots, void* out, int n_tokens,
                                  int nq, int nkv, int D, int page, float scale, int window,
                                  cudaStream_t s) {
  return launch<float>(q, k_pages, v_pages, block_table, max_pages, token_seq, token_pos, slots,
                       out, n_tokens, nq, nkv, D, page, scale, window, s);
}
GB_EXPORT int gb_attn_generic_bf16(const void* q, const void* k_pages, const void* v_pages,
                                   const int* block_table, int max_pages, const int* token_seq,
                                   const int* token_pos, const int* slots, void* out, int n_tokens,
                                   int nq, int nkv, int D, int page, float scale, int window,
                                   cudaStream_t s) {
  return launch<bf16>(q, k_pages, v_pages, block_table, max_pages, token_seq, token_pos, slots,
                      out, n_tokens, nq, nkv, D, page, scale, window, s);
}
