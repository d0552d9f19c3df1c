// Next-token choice on the device, one block per row of 32-bit logits.
//
// gb_argmax_f32: first maximum (ties go to the lowest index, as the reference's
// argmax kernels do, src/kernels.rs:379-385, 502-508).
//
// gb_sample_f32: the reference's sample_next (src/model.rs:2212-2270) without a
// sort of the vocabulary.  s_i = logit_i / temperature; the top_k largest are
// kept (0 < top_k < V; equal scores keep index order); p_i = exp(s_i - max);
// with top_p < 1 the shortest prefix, in descending order, whose normalised
// mass reaches top_p is kept; then u * sum(p) is walked over the kept set.
// "The k-th largest" and "the prefix that reaches top_p" are both thresholds on
// the score, found by a 4-pass radix select over an order-preserving 32-bit key
// (counts for top_k, probability mass for top_p), with ties at the threshold
// resolved by index.  The walk is in index order (the reference walks in
// descending order of probability; the distribution is the same).
// temperature <= 1e-5 falls back to argmax (src/model.rs:2216-2218).
#include "common.cuh"
#include <limits.h>

#define ST 1024

__device__ __forceinline__ uint32_t okey(float s) {
  if (s != s) return 0u;  // NaN sorts below everything
  const uint32_t b = __float_as_uint(s);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
  const uint32_t b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(b);
}

struct ArgBest {
  float v;
  int i;
};
__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

// every thread returns the block's first maximum
__device__ ArgBest block_argmax(const float* row, int V, float mul, ArgBest* sh) {
  ArgBest best{-INFINITY, INT_MAX};
  for (int i = threadIdx.x; i < V; i += ST) {
    float v = row[i] * mul;
    if (v != v) v = -INFINITY;
    if (v > best.v || (v == best.v && i < best.i)) best = ArgBest{v, i};
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = best;
  __syncthreads();
  ArgBest r = sh[0];
  for (int w = 1; w < ST / 32; ++w) r = better(r, sh[w]);
  if (r.i == INT_MAX) r.i = 0;  // a row of NaN or -inf
  return r;
}

// Stage 1: block (chunk, row) finds the first maximum of its slice of the row.
// Stage 2: one warp per row picks the first maximum among the chunks.  Two short
// launches instead of one block per row, which left most of the GPU idle.
#define ARGMAX_CHUNKS 32

__global__ void __launch_bounds__(256) argmax_partial_kernel(const float* logits, int V,
                                                             float* part_v, int* part_i) {
  __shared__ ArgBest sh[8];
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int row = blockIdx.y, chunk = blockIdx.x;
  const int per = (V + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS;
  const int lo = chunk * per, hi = min(V, lo + per);
  const float* r = logits + (size_t)row * V;
  ArgBest best{-INFINITY, INT_MAX};
  for (int i = lo + threadIdx.x; i < hi; i += 256) {
    float v = r[i];
    if (v != v) v = -INFINITY;
    if (v > best.v || (v == best.v && i < best.i)) best = ArgBest{v, i};
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    ArgBest b = sh[0];
    for (int w = 1; w < 8; ++w) b = better(b, sh[w]);
    part_v[row * ARGMAX_CHUNKS + chunk] = b.v;
    part_i[row * ARGMAX_CHUNKS + chunk] = b.i;
  }
}

__global__ void __launch_bounds__(32) argmax_final_kernel(const float* part_v, const int* part_i,
                                                          int* out) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int row = blockIdx.x;
  ArgBest best{part_v[row * ARGMAX_CHUNKS + threadIdx.x], part_i[row * ARGMAX_CHUNKS + threadIdx.x]};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  if (threadIdx.x == 0) out[row] = best.i == INT_MAX ? 0 : best.i;
}

// scratch: n_rows * 32 floats followed by n_rows * 32 ints (the caller's).
GB_EXPORT int gb_argmax_f32(const float* logits, int n_rows, int V, int* out, void* scratch,
                            cudaStream_t s) {
  if (n_rows < 0 || V <= 0 || !scratch) return GB_ERR_BAD_ARG;
  if (n_rows == 0) return 0;
  if (n_rows > 65535) return GB_ERR_UNSUPPORTED;
  float* pv = (float*)scratch;
  int* pi = (int*)(pv + (size_t)n_rows * ARGMAX_CHUNKS);
  int e = gb_launch(argmax_partial_kernel, dim3(ARGMAX_CHUNKS, n_rows), dim3(256), 0, s, logits, V,
                    pv, pi);
  if (e) return e;
  return gb_launch(argmax_final_kernel, dim3(n_rows), dim3(32), 0, s, (const float*)pv,
                   (const int*)pi, out);
}

// ---------------------------------------------------------------------------
struct Members {       // i is kept when key > thr, or key == thr and i <= cut
  uint32_t thr;
  int cut;
};
__device__ __forceinline__ bool member(const Members& m, uint32_t key, int i) {
  return key > m.thr || (key == m.thr && i <= m.cut);
}

__device__ double block_sum_f64(double v, double* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  double r = 0.0;
  for (int w = 0; w < ST / 32; ++w) r += sh[w];
  return r;
}

// Inclusive scan of one value per thread over the block; returns the thread's
// inclusive prefix and the block total.
template <typename T>
__device__ T block_scan(T v, T* sh, T* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    T n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += n;
  }
  __syncthreads();
  if (lane == 31) sh[warp] = v;
  __syncthreads();
  T before = 0, all = 0;
  for (int w = 0; w < ST / 32; ++w) {
    if (w < warp) before += sh[w];
    all += sh[w];
  }
  *total = all;
  return v + before;
}

struct Shared {
  unsigned int cnt[256];
  double mass[256];
  ArgBest best[ST / 32];
  double red[ST / 32];
  int ired[ST / 32];
  uint32_t sel_prefix;
  unsigned int sel_count;   // elements in the chosen bin
  double rest_mass;         // mass still wanted inside the chosen bin
  unsigned int rest_count;  // rank still wanted inside the chosen bin
  int found;
};

// The index of the r-th element (1-based, index order) whose key equals `key`
// among the members of `base`.
__device__ int find_tie_cut(const float* row, int V, float inv_t, const Members& base, uint32_t key,
                            unsigned int r, Shared& sh) {
  unsigned int seen = 0;
  if (threadIdx.x == 0) sh.found = INT_MAX;
  __syncthreads();
  for (int c = 0; c < V; c += ST) {
    const int i = c + threadIdx.x;
    int flag = 0;
    if (i < V) {
      const uint32_t k = okey(row[i] * inv_t);
      flag = (k == key && member(base, k, i)) ? 1 : 0;
    }
    int total;
    const int incl = block_scan<int>(flag, sh.ired, &total);
    if (flag && seen + incl == r) sh.found = i;
    seen += total;
    __syncthreads();
    if (seen >= r) break;
  }
  __syncthreads();
  return sh.found;
}

__global__ void __launch_bounds__(ST)
sample_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ u, int* __restrict__ out) {
  __shared__ Shared sh;
  const int b = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (size_t)b * V;
  const float temp = temperature[b];
  if (!(temp > 1.0e-5f)) {
    const ArgBest r = block_argmax(row, V, 1.0f, sh.best);
    if (tid == 0) out[b] = r.i;
    return;
  }
  const float inv_t = 1.0f / temp;
  const ArgBest top = block_argmax(row, V, inv_t, sh.best);
  const float smax = top.v;
  int K = top_k[b];
  float P = top_p[b];
  P = fminf(fmaxf(P, 0.f), 1.f);

  Members mem{0u, INT_MAX};

  // ---- top-k: the k-th largest key, by counts --------------------------------
  if (K > 0 && K < V) {
    uint32_t prefix = 0;
    unsigned int want = (unsigned int)K;
    unsigned int eq = 0;
    for (int d = 3; d >= 0; --d) {
      for (int j = tid; j < 256; j += ST) sh.cnt[j] = 0;
      __syncthreads();
      const int shift = 8 * d;
      for (int i = tid; i < V; i += ST) {
        const uint32_t k = okey(row[i] * inv_t);
        if (d == 3 || (k >> (shift + 8)) == (prefix >> (shift + 8)))
          atomicAdd(&sh.cnt[(k >> shift) & 255u], 1u);
      }
      __syncthreads();
      if (tid == 0) {
        unsigned int w = want;
        int bin = 0;
        for (int j = 255; j >= 0; --j) {
          if (w <= sh.cnt[j]) { bin = j; break; }
          w -= sh.cnt[j];
        }
        sh.sel_prefix = prefix | ((uint32_t)bin << shift);
        sh.rest_count = w;
        sh.sel_count = sh.cnt[bin];
      }
      __syncthreads();
      prefix = sh.sel_prefix;
      want = sh.rest_count;
      eq = sh.sel_count;
      __syncthreads();
    }
    mem.thr = prefix;
    if (want < eq) mem.cut = find_tie_cut(row, V, inv_t, Members{0u, INT_MAX}, prefix, want, sh);
  }

  // ---- mass of the kept set ---------------------------------------------------
  double local = 0.0;
  for (int i = tid; i < V; i += ST) {
    const float s = row[i] * inv_t;
    const uint32_t k = okey(s);
    if (member(mem, k, i)) local += (double)expf(s - smax);
  }
  double total = block_sum_f64(local, sh.red);

  // ---- top-p: the key at which the descending cumulative mass reaches P * total
  if (P < 1.0f) {
    uint32_t prefix = 0;
    double want = (double)P * total;
    unsigned int eq = 0;
    for (int d = 3; d >= 0; --d) {
      for (int j = tid; j < 256; j += ST) { sh.cnt[j] = 0; sh.mass[j] = 0.0; }
      __syncthreads();
      const int shift = 8 * d;
      for (int i = tid; i < V; i += ST) {
        const float s = row[i] * inv_t;
        const uint32_t k = okey(s);
        if (member(mem, k, i) && (d == 3 || (k >> (shift + 8)) == (prefix >> (shift + 8)))) {
          atomicAdd(&sh.cnt[(k >> shift) & 255u], 1u);
          atomicAdd(&sh.mass[(k >> shift) & 255u], (double)expf(s - smax));
        }
      }
      __syncthreads();
      if (tid == 0) {
        double w = want;
        int bin = -1, lowest = 0;
        for (int j = 255; j >= 0; --j) {
          if (!sh.cnt[j]) continue;
          lowest = j;
          if (sh.mass[j] >= w) { bin = j; break; }
          w -= sh.mass[j];
        }
        if (bin < 0) { bin = lowest; w = sh.mass[lowest]; }  // rounding left a crumb: keep all
        sh.sel_prefix = prefix | ((uint32_t)bin << shift);
        sh.rest_mass = w;
        sh.sel_count = sh.cnt[bin];
      }
      __syncthreads();
      prefix = sh.sel_prefix;
      want = sh.rest_mass;
      eq = sh.sel_count;
      __syncthreads();
    }
    // `want` is the mass still needed from the eq elements equal to the threshold
    const double pv = (double)expf(key_to_float(prefix) - smax);
    unsigned int r = eq;
    if (pv > 0.0) {
      const double need = ceil(want / pv);
      r = need < 1.0 ? 1u : (need > (double)eq ? eq : (unsigned int)need);
    }
    Members narrowed{prefix, INT_MAX};
    // ties at a shared threshold obey the tighter of the two limits
    if (prefix == mem.thr && mem.cut != INT_MAX) {
      narrowed.cut = mem.cut;
      // r counts members only; find_tie_cut below counts members of `mem` too
    }
    if (r < eq) {
      const int cut = find_tie_cut(row, V, inv_t, mem, prefix, r, sh);
      narrowed.cut = cut < narrowed.cut ? cut : narrowed.cut;
    }
    mem = narrowed;
    local = 0.0;
    for (int i = tid; i < V; i += ST) {
      const float s = row[i] * inv_t;
      const uint32_t k = okey(s);
      if (member(mem, k, i)) local += (double)expf(s - smax);
    }
    total = block_sum_f64(local, sh.red);
  }

  if (!(total > 0.0) || total != total || isinf(total)) {  // src/model.rs:2260-2263
    if (tid == 0) out[b] = top.i;
    return;
  }

  // ---- the draw: first index whose running mass reaches u * total --------------
  const double threshold = (double)u[b] * total;
  double seen = 0.0;
  if (tid == 0) sh.found = INT_MAX;
  __syncthreads();
  int last_member = -1;
  for (int c = 0; c < V; c += ST) {
    const int i = c + tid;
    double p = 0.0;
    bool in = false;
    if (i < V) {
      const float s = row[i] * inv_t;
      const uint32_t k = okey(s);
      in = member(mem, k, i);
      if (in) p = (double)expf(s - smax);
    }
    if (in) last_member = i;
    double ctotal;
    const double incl = block_scan<double>(p, sh.red, &ctotal);
    if (in && seen + incl >= threshold) atomicMin(&sh.found, i);
    seen += ctotal;
    __syncthreads();
    if (sh.found != INT_MAX) break;
  }
  __syncthreads();
  int token = sh.found;
  if (token == INT_MAX) {  // rounding left the threshold above the last sum
    int lm = last_member;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lm = max(lm, __shfl_xor_sync(0xffffffffu, lm, o));
    __syncthreads();
    if ((tid & 31) == 0) sh.ired[tid >> 5] = lm;
    __syncthreads();
    if (tid == 0) {
      int best = -1;
      for (int w = 0; w < ST / 32; ++w) best = max(best, sh.ired[w]);
      sh.found = best < 0 ? top.i : best;
    }
    __syncthreads();
    token = sh.found;
  }
  if (tid == 0) out[b] = token;
}

GB_EXPORT int gb_sample_f32(const float* logits, int n_rows, int V, const float* temperature,
                            const int* top_k, const float* top_p, const float* u, int* out,
                            cudaStream_t s) {
  if (n_rows < 0 || V <= 0 || !temperature || !top_k || !top_p || !u) return GB_ERR_BAD_ARG;
  if (n_rows == 0) return 0;
  sample_kernel<<<n_rows, ST, 0, s>>>(logits, V, temperature, top_k, top_p, u, out);
  return gb_status();
}
