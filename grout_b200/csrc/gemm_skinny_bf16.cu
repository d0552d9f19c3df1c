// Decode-time linear layer: y[M, N] = x[M, K] . W[N, K]^T for a handful of rows
// (M <= 64), bf16 in, 32-bit accumulate, bf16 or 32-bit out.  The product is
// bound by reading W once, so the kernel is built around the weight stream:
// every lane issues 16-byte loads straight from global memory into the operand
// registers of mma.sync.m16n8k16, with the weight rows as the 16-row operand
// and the few activation rows as the 8-wide one ("swap A/B").  Where the
// reference calls cuBLAS GEMV (src/cublas.rs:572-667, called per projection at
// src/model.rs:3170-3176), this streams the weights itself.
//
// k order inside one MMA is permuted (a lane feeds 8 consecutive k of its row to
// two MMAs); A and B use the same permutation, so the dot products are exact
// sums over all k.
//
// Parallelism.  A block of four warps owns a tile of weight rows and one slice
// of K; its warps take the slice's 32-element chunks in turn and are summed in
// warp order.  When N is small the grid is widened by splitting K over
// `ksplit` blocks per tile so that enough loads are in flight to cover DRAM
// latency.  Each block then writes its 32-bit partial tile to scratch and bumps
// the tile's counter; the block that arrives last adds the partials in split
// order 0..ksplit-1 and writes the output.  No block waits for another, and the
// order of every sum is fixed by (N, K, M's bucket) alone, never by timing.
// The counter is left at zero for the next launch.
//
// Epilogue variant SILU: the weight rows are gate and up projections interleaved
// in groups of 8 (rows 16t..16t+7 gate, 16t+8..16t+15 up, for the same 8
// intermediate features), and the kernel writes silu(gate) * up, N / 2 columns
// (the reference's silu_mul_2d_f16, src/kernels.rs:271-296, as an epilogue).
#include "common.cuh"

#define SK_WARPS 4
#define SK_THREADS (SK_WARPS * 32)

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct SkinnyArgs {
  const bf16* x;       // [M, K]
  const bf16* W;       // [N, K]
  void* y;             // [M, N] or, with SILU, [M, N / 2]
  float* scratch;      // [tiles, ksplit, 8 NT, 16 MT]   (ksplit > 1)
  unsigned* counters;  // [tiles], zero before the first launch   (ksplit > 1)
  int M, N, K, ksplit, chunks_per_split;
};

// NT: activation rows in tiles of 8; MT: weight rows in tiles of 16 per block.
template <int NT, int MT, int UNROLL, typename OutT, bool SILU>
__global__ void __launch_bounds__(SK_THREADS) skinny_kernel(const SkinnyArgs a) {
  constexpr int ROWS = 16 * MT, COLS = 8 * NT;
  __shared__ float red[COLS][ROWS + 1];
  __shared__ int is_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int tile = blockIdx.x, split = blockIdx.y;
  const int r0 = tile * ROWS;
  const int M = a.M, N = a.N, K = a.K;

  float acc[MT][NT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

  const bf16* wrow[MT][2];
  bool wok[MT][2];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int r = r0 + i * 16 + g + hf * 8;
      wok[i][hf] = r < N;
      wrow[i][hf] = a.W + (size_t)(r < N ? r : N - 1) * K;
    }
  const bf16* xrow[NT];
  bool xok[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int m = j * 8 + g;
    xok[j] = m < M;
    xrow[j] = a.x + (size_t)(m < M ? m : M - 1) * K;
  }

  const int nchunks = (K + 31) / 32;
  const int c_begin = split * a.chunks_per_split;
  const int c_end = min(nchunks, c_begin + a.chunks_per_split);
  // UNROLL chunks are fetched before any of them is multiplied, so that a warp
  // keeps UNROLL * (2 MT + NT) 16-byte loads in flight.  The first batch of
  // weights is requested before the kernel waits for its producer: weights are
  // no kernel's output, the activations are.
  bool waited = false;
  for (int c = c_begin + warp; c < c_end || !waited; c += SK_WARPS * UNROLL) {
    uint4 wv[UNROLL][MT][2], xv[UNROLL][NT];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int cu = c + u * SK_WARPS;
      const int k = cu * 32 + t * 8;
      const bool kok = cu < c_end && k < K;  // K is a multiple of 8: all 8 elements are inside
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf)
          wv[u][i][hf] = (kok && wok[i][hf]) ? ld_stream(wrow[i][hf] + k) : make_uint4(0, 0, 0, 0);
    }
    if (!waited) {
      pdl_wait();
      waited = true;
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int cu = c + u * SK_WARPS;
      const int k = cu * 32 + t * 8;
      const bool kok = cu < c_end && k < K;
#pragma unroll
      for (int j = 0; j < NT; ++j)
        xv[u][j] = (kok && xok[j]) ? __ldcg(reinterpret_cast<const uint4*>(xrow[j] + k))
                                   : make_uint4(0, 0, 0, 0);   // written by the producer: read at L2
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          mma_bf16(acc[i][j], wv[u][i][0].x, wv[u][i][1].x, wv[u][i][0].y, wv[u][i][1].y,
                   xv[u][j].x, xv[u][j].y);
          mma_bf16(acc[i][j], wv[u][i][0].z, wv[u][i][1].z, wv[u][i][0].w, wv[u][i][1].w,
                   xv[u][j].z, xv[u][j].w);
        }
  }

  pdl_launch_dependents();   // the weight stream of this block is over

  // sum the warps' partial tiles in warp order
  for (int w = 0; w < SK_WARPS; ++w) {
    if (warp == w) {
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int row = i * 16 + g + (e >> 1) * 8;   // weight row inside the tile
            const int col = j * 8 + t * 2 + (e & 1);     // activation row
            if (w == 0) red[col][row] = acc[i][j][e];
            else red[col][row] += acc[i][j][e];
          }
    }
    __syncthreads();
  }

  if (a.ksplit > 1) {
    float* mine = a.scratch + ((size_t)tile * a.ksplit + split) * (ROWS * COLS);
    for (int e = threadIdx.x; e < ROWS * M; e += SK_THREADS) mine[e] = red[e / ROWS][e % ROWS];
    __threadfence();   // the partial is visible before the counter moves
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned old = atomicAdd(&a.counters[tile], 1u);
      is_last = (old == (unsigned)a.ksplit - 1u);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();   // see the other blocks' partials
    const float* all = a.scratch + (size_t)tile * a.ksplit * (ROWS * COLS);
    for (int e = threadIdx.x; e < ROWS * M; e += SK_THREADS) {
      float s = 0.f;
      for (int sp = 0; sp < a.ksplit; ++sp) s += __ldcg(all + (size_t)sp * (ROWS * COLS) + e);
      red[e / ROWS][e % ROWS] = s;
    }
    if (threadIdx.x == 0) a.counters[tile] = 0u;   // ready for the next launch
    __syncthreads();
  }

  OutT* y = (OutT*)a.y;
  if (SILU) {
    // rows 16q..16q+7 of the tile are gates, 16q+8..16q+15 the matching ups
    const int n_out = N / 2;
    for (int e = threadIdx.x; e < (ROWS / 2) * M; e += SK_THREADS) {
      const int pr = e % (ROWS / 2), col = e / (ROWS / 2);
      const int row = (pr / 8) * 16 + (pr % 8);
      const int feat = r0 / 2 + pr;
      if (feat < n_out) {
        const float gt = red[col][row], up = red[col][row + 8];
        y[(size_t)col * n_out + feat] = from_f32<OutT>(gt / (1.0f + expf(-gt)) * up);
      }
    }
  } else {
    for (int e = threadIdx.x; e < ROWS * M; e += SK_THREADS) {
      const int row = e % ROWS, col = e / ROWS;
      if (r0 + row < N) y[(size_t)col * N + r0 + row] = from_f32<OutT>(red[col][row]);
    }
  }
}

template <int NT, int MT, int UNROLL, typename OutT, bool SILU>
static int launch(const SkinnyArgs& a, cudaStream_t s) {
  const int rows = 16 * MT;
  dim3 grid((a.N + rows - 1) / rows, a.ksplit);
  return gb_launch(skinny_kernel<NT, MT, UNROLL, OutT, SILU>, grid, dim3(SK_THREADS), 0, s, a);
}

template <typename OutT, bool SILU>
static int dispatch(const SkinnyArgs& a, cudaStream_t s) {
  if (a.M <= 8) return launch<1, 1, 8, OutT, SILU>(a, s);
  if (a.M <= 16) return launch<2, 1, 4, OutT, SILU>(a, s);
  if (a.M <= 32) return launch<4, 2, 2, OutT, SILU>(a, s);
  return launch<8, 2, 2, OutT, SILU>(a, s);
}

// Weight rows per tile for M activation rows (the host sizes grid and scratch with it).
GB_EXPORT int gb_gemm_skinny_tile_rows(int M) { return M <= 16 ? 16 : 32; }
GB_EXPORT int gb_gemm_skinny_tile_cols(int M) { return M <= 8 ? 8 : (M <= 16 ? 16 : (M <= 32 ? 32 : 64)); }

// out_f32: 1 writes 32-bit outputs (logits), 0 writes bf16.
// silu: 1 for the interleaved gate|up epilogue (then N must be a multiple of 16).
GB_EXPORT int gb_gemm_skinny_bf16(const SkinnyArgs* a, int out_f32, int silu, cudaStream_t s) {
  if (a->M < 0 || a->N <= 0 || a->K <= 0 || a->ksplit <= 0 || a->chunks_per_split <= 0)
    return GB_ERR_BAD_ARG;
  if (a->M > 64) return GB_ERR_UNSUPPORTED;
  if (a->K % 8) return GB_ERR_UNSUPPORTED;  // rows must start on 16-byte boundaries
  if (silu && (a->N % 16)) return GB_ERR_UNSUPPORTED;
  if ((((uintptr_t)a->x) | ((uintptr_t)a->W)) & 15) return GB_ERR_BAD_ARG;
  if (a->ksplit > 1 && (!a->scratch || !a->counters)) return GB_ERR_BAD_ARG;
  if ((long long)a->ksplit * a->chunks_per_split < (a->K + 31) / 32) return GB_ERR_BAD_ARG;
  if (a->ksplit > 65535) return GB_ERR_BAD_ARG;
  if (a->M == 0) return 0;
  if (silu) return out_f32 ? dispatch<float, true>(*a, s) : dispatch<bf16, true>(*a, s);
  return out_f32 ? dispatch<float, false>(*a, s) : dispatch<bf16, false>(*a, s);
}

// ---------------------------------------------------------------------------
// The same product for callers that cannot allocate: see gemm_skinny_noalloc.h.
// The scratch is the two static device arrays below; in host code their names
// stand for the symbols, not for device addresses, so the addresses are looked
// up once per device and passed to the kernel like any other pointer.
#include <mutex>
#include "gemm_skinny_noalloc.h"

static __device__ __align__(256) float gb_noalloc_scratch[GB_NOALLOC_SCRATCH_FLOATS];
static __device__ __align__(256) unsigned gb_noalloc_counters[GB_NOALLOC_MAX_TILES];

struct NoAllocDevice {
  float* scratch = nullptr;
  unsigned* counters = nullptr;
  int sm_count = 0;
  bool ready = false;
};
static NoAllocDevice g_noalloc[GB_NOALLOC_MAX_DEVICES];
static std::mutex g_noalloc_mutex;

// Once per device, with that device current.
static int noalloc_setup(int dev, NoAllocDevice** out) {
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  NoAllocDevice& d = g_noalloc[dev];
  if (!d.ready) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, gb_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    d.scratch = (float*)p;
    e = cudaGetSymbolAddress(&p, gb_noalloc_counters);
    if (e != cudaSuccess) return (int)e;
    d.counters = (unsigned*)p;
    e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
    d.ready = true;
  }
  *out = &d;
  return 0;
}

GB_EXPORT int gb_gemm_skinny_bf16_noalloc(const void* x, const void* W, void* y, int M, int N,
                                          int K, int out_f32, cudaStream_t stream) {
  if (M < 0 || N <= 0 || K <= 0 || !x || !W || !y) return GB_ERR_BAD_ARG;
  if (M > 64 || (K % 8)) return GB_ERR_UNSUPPORTED;
  if ((((uintptr_t)x) | ((uintptr_t)W)) & 15) return GB_ERR_BAD_ARG;
  if (M == 0) return 0;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= GB_NOALLOC_MAX_DEVICES) return GB_ERR_UNSUPPORTED;
  NoAllocDevice* d = nullptr;
  int rc = noalloc_setup(dev, &d);
  if (rc) return rc;

  // the split the allocating path uses: about eight blocks per SM, at least 16
  // chunks of 32 elements per block, at most 16 splits
  const int rows = gb_gemm_skinny_tile_rows(M), cols = gb_gemm_skinny_tile_cols(M);
  const int tiles = (N + rows - 1) / rows;
  const int nchunks = (K + 31) / 32;
  int ks = (8 * d->sm_count + tiles - 1) / tiles;
  if (ks > nchunks / 16) ks = nchunks / 16;
  if (ks > 16) ks = 16;
  if (ks < 1) ks = 1;
  const int per = (nchunks + ks - 1) / ks;
  ks = (nchunks + per - 1) / per;

  SkinnyArgs a;
  a.x = (const bf16*)x;
  a.W = (const bf16*)W;
  a.y = y;
  a.scratch = nullptr;
  a.counters = nullptr;
  a.M = M;
  a.N = N;
  a.K = K;
  a.ksplit = ks;
  a.chunks_per_split = per;
  if (ks > 1) {
    if (tiles > GB_NOALLOC_MAX_TILES ||
        (long long)tiles * ks * rows * cols > (long long)GB_NOALLOC_SCRATCH_FLOATS)
      return GB_ERR_TOO_LARGE;
    a.scratch = d->scratch;
    a.counters = d->counters;
    // the array keeps the last call's contents: the counters must start at zero
    e = cudaMemsetAsync(d->counters, 0, (size_t)tiles * sizeof(unsigned), stream);
    if (e != cudaSuccess) return (int)e;
  }
  return out_f32 ? dispatch<float, false>(a, stream) : dispatch<bf16, false>(a, stream);
}
