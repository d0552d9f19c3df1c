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
// Work split ("stream-K").  The weight matrix is cut into tiles of ROWS weight
// rows and each tile's K into chunks of 32 elements; tile-major, chunk-minor,
// that is one line of U = tiles * chunks units of equal cost.  The grid is
// exactly as many blocks as the GPU holds at once (occupancy x SMs), and block p
// streams the units [p U / P, (p+1) U / P): every SM reads the same number of
// bytes and there is no last, half-empty wave.  A block that covers a tile's
// whole K writes the output; a tile shared by several blocks is finished by the
// one that arrives last (a counter per tile): the others leave their 32-bit
// partial in scratch, the last adds them in block order and writes.  No block
// waits for another, and the order of every sum is fixed by (N, K, M's bucket,
// the GPU's size), never by timing.  Counters are left at zero.
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
  float* scratch;      // [2 * blocks][8 NT * 16 MT]: a block's first and last partial tile
  unsigned* counters;  // [tiles], zero before the first launch
  int M, N, K;
};

// The block that streams unit u when U units are dealt to P blocks in spans
// [p U / P, (p + 1) U / P).
__device__ __forceinline__ int block_of_unit(long long u, long long U, int P) {
  return (int)(((u + 1) * P - 1) / U);
}

// NT: activation rows in tiles of 8; MT: weight rows in tiles of 16 per tile.
template <int NT, int MT, int UNROLL, typename OutT, bool SILU>
__global__ void __launch_bounds__(SK_THREADS) skinny_kernel(const SkinnyArgs a) {
  constexpr int ROWS = 16 * MT, COLS = 8 * NT, TILE = ROWS * COLS;
  __shared__ float red[COLS][ROWS + 1];
  __shared__ int is_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int M = a.M, N = a.N, K = a.K;
  const int P = gridDim.x, p = blockIdx.x;
  const int nchunks = (K + 31) / 32;
  const int tiles = (N + ROWS - 1) / ROWS;
  const long long U = (long long)tiles * nchunks;
  const long long u_begin = p * U / P, u_end = (p + 1) * U / P;

  const bf16* xrow[NT];
  bool xok[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int m = j * 8 + g;
    xok[j] = m < M;
    xrow[j] = a.x + (size_t)(m < M ? m : M - 1) * K;
  }

  bool waited = false;
  for (long long u = u_begin; u < u_end;) {
    const int tile = (int)(u / nchunks);
    const int c_lo = (int)(u - (long long)tile * nchunks);
    const int c_hi = (int)min((long long)nchunks, c_lo + (u_end - u));
    u += c_hi - c_lo;
    const int r0 = tile * ROWS;

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
    float acc[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

    // UNROLL chunks are fetched before any of them is multiplied, so that a warp
    // keeps UNROLL * (2 MT + NT) 16-byte loads in flight.  The very first batch
    // of weights is requested before the kernel waits for its producer: weights
    // are no kernel's output, the activations are.
    for (int c = c_lo + warp; c < c_hi || !waited; c += SK_WARPS * UNROLL) {
      uint4 wv[UNROLL][MT][2], xv[UNROLL][NT];
#pragma unroll
      for (int uu = 0; uu < UNROLL; ++uu) {
        const int cu = c + uu * SK_WARPS;
        const int k = cu * 32 + t * 8;
        const bool kok = cu < c_hi && k < K;  // K is a multiple of 8: all 8 elements are inside
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
          for (int hf = 0; hf < 2; ++hf)
            wv[uu][i][hf] =
                (kok && wok[i][hf]) ? ld_stream(wrow[i][hf] + k) : make_uint4(0, 0, 0, 0);
      }
      if (!waited) {
        pdl_wait();
        waited = true;
      }
#pragma unroll
      for (int uu = 0; uu < UNROLL; ++uu) {
        const int cu = c + uu * SK_WARPS;
        const int k = cu * 32 + t * 8;
        const bool kok = cu < c_hi && k < K;
#pragma unroll
        for (int j = 0; j < NT; ++j)  // written by the producer kernel: read at L2
          xv[uu][j] = (kok && xok[j]) ? __ldcg(reinterpret_cast<const uint4*>(xrow[j] + k))
                                      : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int uu = 0; uu < UNROLL; ++uu)
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            mma_bf16(acc[i][j], wv[uu][i][0].x, wv[uu][i][1].x, wv[uu][i][0].y, wv[uu][i][1].y,
                     xv[uu][j].x, xv[uu][j].y);
            mma_bf16(acc[i][j], wv[uu][i][0].z, wv[uu][i][1].z, wv[uu][i][0].w, wv[uu][i][1].w,
                     xv[uu][j].z, xv[uu][j].w);
          }
    }
    if (u >= u_end) pdl_launch_dependents();   // this block's weight stream is over

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

    bool write_out = true;
    if (c_lo != 0 || c_hi != nchunks) {
      // a shared tile: leave the partial; the block that arrives last adds them up
      const long long t0 = (long long)tile * nchunks;
      const int p_first = block_of_unit(t0, U, P), p_last = block_of_unit(t0 + nchunks - 1, U, P);
      const bool my_first_tile = (int)(u_begin / nchunks) == tile;
      float* mine = a.scratch + ((size_t)2 * p + (my_first_tile ? 0 : 1)) * TILE;
      for (int e = threadIdx.x; e < ROWS * M; e += SK_THREADS) mine[e] = red[e / ROWS][e % ROWS];
      __threadfence();   // the partial is visible before the counter moves
      __syncthreads();
      if (threadIdx.x == 0) {
        const unsigned old = atomicAdd(&a.counters[tile], 1u);
        is_last = (old == (unsigned)(p_last - p_first));
      }
      __syncthreads();
      write_out = is_last;
      if (write_out) {
        __threadfence();   // see the other blocks' partials
        for (int e = threadIdx.x; e < ROWS * M; e += SK_THREADS) {
          float s = 0.f;
          for (int q = p_first; q <= p_last; ++q) {
            const bool q_first_tile = (int)(((long long)q * U / P) / nchunks) == tile;
            s += __ldcg(a.scratch + ((size_t)2 * q + (q_first_tile ? 0 : 1)) * TILE + e);
          }
          red[e / ROWS][e % ROWS] = s;
        }
        if (threadIdx.x == 0) a.counters[tile] = 0u;   // ready for the next launch
        __syncthreads();
      }
    }

    if (write_out) {
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
    __syncthreads();   // red is reused by the next tile
  }
}

// How a launch is laid out: blocks, scratch floats, counters.
struct SkinnyPlan {
  int blocks, scratch_floats, counters;
};

template <int NT, int MT, int UNROLL, typename OutT, bool SILU>
static int plan_for(int N, int K, SkinnyPlan* plan) {
  static int per_sm = 0, sms = 0;   // per instantiation; the same on every device of a host
  if (!per_sm) {
    int dev = 0, n = 0, s = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess)
      e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(
          &n, skinny_kernel<NT, MT, UNROLL, OutT, SILU>, SK_THREADS, 0);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&s, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
    if (n < 1 || s < 1) return GB_ERR_UNSUPPORTED;
    per_sm = n;
    sms = s;
  }
  const int rows = 16 * MT, cols = 8 * NT;
  const long long units = (long long)((N + rows - 1) / rows) * ((K + 31) / 32);
  long long blocks = (long long)per_sm * sms;
  if (blocks > units) blocks = units;
  plan->blocks = (int)blocks;
  plan->scratch_floats = (int)(2 * blocks * rows * cols);
  plan->counters = (N + rows - 1) / rows;
  return 0;
}

template <int NT, int MT, int UNROLL, typename OutT, bool SILU>
static int run(const SkinnyArgs* a, SkinnyPlan* plan, cudaStream_t s) {
  SkinnyPlan pl;
  int e = plan_for<NT, MT, UNROLL, OutT, SILU>(a->N, a->K, &pl);
  if (e) return e;
  if (plan) {   // planning only
    *plan = pl;
    return 0;
  }
  return gb_launch(skinny_kernel<NT, MT, UNROLL, OutT, SILU>, dim3(pl.blocks), dim3(SK_THREADS), 0, s,
                   *a);
}

template <typename OutT, bool SILU>
static int dispatch(const SkinnyArgs* a, SkinnyPlan* plan, cudaStream_t s) {
  if (a->M <= 8) return run<1, 1, 8, OutT, SILU>(a, plan, s);
  if (a->M <= 16) return run<2, 1, 4, OutT, SILU>(a, plan, s);
  if (a->M <= 32) return run<4, 2, 2, OutT, SILU>(a, plan, s);
  return run<8, 2, 2, OutT, SILU>(a, plan, s);
}

static int dispatch_all(const SkinnyArgs* a, int out_f32, int silu, SkinnyPlan* plan,
                        cudaStream_t s) {
  if (silu) return out_f32 ? dispatch<float, true>(a, plan, s) : dispatch<bf16, true>(a, plan, s);
  return out_f32 ? dispatch<float, false>(a, plan, s) : dispatch<bf16, false>(a, plan, s);
}

static int check_shape(int M, int N, int K, int silu) {
  if (M < 0 || N <= 0 || K <= 0) return GB_ERR_BAD_ARG;
  if (M > 64) return GB_ERR_UNSUPPORTED;
  if (K % 8) return GB_ERR_UNSUPPORTED;  // rows must start on 16-byte boundaries
  if (silu && (N % 16)) return GB_ERR_UNSUPPORTED;
  return 0;
}

// What a launch for this shape needs: plan[0] blocks, plan[1] scratch floats,
// plan[2] counters (32-bit, zero before the first launch).  Call it with the
// device current; it launches nothing.
GB_EXPORT int gb_gemm_skinny_plan(int M, int N, int K, int out_f32, int silu, int* plan) {
  int e = check_shape(M, N, K, silu);
  if (e) return e;
  SkinnyArgs a = {};
  a.M = M > 0 ? M : 1;
  a.N = N;
  a.K = K;
  SkinnyPlan pl;
  e = dispatch_all(&a, out_f32, silu, &pl, 0);
  if (e) return e;
  plan[0] = pl.blocks;
  plan[1] = pl.scratch_floats;
  plan[2] = pl.counters;
  return 0;
}

// out_f32: 1 writes 32-bit outputs (logits), 0 writes bf16.
// silu: 1 for the interleaved gate|up epilogue (then N must be a multiple of 16).
// scratch and counters must hold what gb_gemm_skinny_plan reports.
GB_EXPORT int gb_gemm_skinny_bf16(const SkinnyArgs* a, int out_f32, int silu, cudaStream_t s) {
  int e = check_shape(a->M, a->N, a->K, silu);
  if (e) return e;
  if ((((uintptr_t)a->x) | ((uintptr_t)a->W)) & 15) return GB_ERR_BAD_ARG;
  if (!a->scratch || !a->counters) return GB_ERR_BAD_ARG;
  if (a->M == 0) return 0;
  return dispatch_all(a, out_f32, silu, nullptr, s);
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
    d.ready = true;
  }
  *out = &d;
  return 0;
}

GB_EXPORT int gb_gemm_skinny_bf16_noalloc(const void* x, const void* W, void* y, int M, int N,
                                          int K, int out_f32, cudaStream_t stream) {
  if (!x || !W || !y) return GB_ERR_BAD_ARG;
  int rc = check_shape(M, N, K, 0);
  if (rc) return rc;
  if ((((uintptr_t)x) | ((uintptr_t)W)) & 15) return GB_ERR_BAD_ARG;
  if (M == 0) return 0;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= GB_NOALLOC_MAX_DEVICES) return GB_ERR_UNSUPPORTED;
  NoAllocDevice* d = nullptr;
  rc = noalloc_setup(dev, &d);
  if (rc) return rc;

  SkinnyArgs a = {};
  a.x = (const bf16*)x;
  a.W = (const bf16*)W;
  a.y = y;
  a.M = M;
  a.N = N;
  a.K = K;
  SkinnyPlan pl;
  rc = dispatch_all(&a, out_f32, 0, &pl, stream);   // the layout the allocating path uses
  if (rc) return rc;
  if (pl.counters > GB_NOALLOC_MAX_TILES || pl.scratch_floats > GB_NOALLOC_SCRATCH_FLOATS)
    return GB_ERR_TOO_LARGE;
  a.scratch = d->scratch;
  a.counters = d->counters;
  // the array keeps the last call's contents: the counters must start at zero
  e = cudaMemsetAsync(d->counters, 0, (size_t)pl.counters * sizeof(unsigned), stream);
  if (e != cudaSuccess) return (int)e;
  return dispatch_all(&a, out_f32, 0, nullptr, stream);
}
