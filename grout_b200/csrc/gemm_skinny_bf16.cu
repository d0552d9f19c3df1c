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
// sums over all k.  The 8 warps of a block split K in interleaved 32-element
// chunks and are summed in warp order, which fixes the order of every output's
// sum independently of M.
#include "common.cuh"

#define SK_WARPS 8

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT: activation rows in tiles of 8; MT: weight rows in tiles of 16 per block.
template <int NT, int MT, typename OutT>
__global__ void __launch_bounds__(SK_WARPS * 32)
skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W, OutT* __restrict__ y, int M,
              int N, int K) {
  constexpr int ROWS = 16 * MT, COLS = 8 * NT;
  __shared__ float red[COLS][ROWS + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int r0 = blockIdx.x * ROWS;

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
      wrow[i][hf] = W + (size_t)(r < N ? r : N - 1) * K;
    }
  const bf16* xrow[NT];
  bool xok[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int m = j * 8 + g;
    xok[j] = m < M;
    xrow[j] = x + (size_t)(m < M ? m : M - 1) * K;
  }

  const int nchunks = (K + 31) / 32;
#pragma unroll 4
  for (int c = warp; c < nchunks; c += SK_WARPS) {
    const int k = c * 32 + t * 8;
    const bool kok = k < K;  // K is a multiple of 8, so the 8 elements are all inside
    uint4 wv[MT][2], xv[NT];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf)
        wv[i][hf] = (kok && wok[i][hf]) ? ld_stream(wrow[i][hf] + k) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int j = 0; j < NT; ++j)
      xv[j] = (kok && xok[j]) ? __ldg(reinterpret_cast<const uint4*>(xrow[j] + k))
                              : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        mma_bf16(acc[i][j], wv[i][0].x, wv[i][1].x, wv[i][0].y, wv[i][1].y, xv[j].x, xv[j].y);
        mma_bf16(acc[i][j], wv[i][0].z, wv[i][1].z, wv[i][0].w, wv[i][1].w, xv[j].z, xv[j].w);
      }
  }

  // sum the warps' partial tiles in warp order
  for (int w = 0; w < SK_WARPS; ++w) {
    if (warp == w) {
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int row = i * 16 + g + (e >> 1) * 8;   // weight row inside the block
            const int col = j * 8 + t * 2 + (e & 1);     // activation row
            if (w == 0) red[col][row] = acc[i][j][e];
            else red[col][row] += acc[i][j][e];
          }
    }
    __syncthreads();
  }
  for (int e = threadIdx.x; e < ROWS * COLS; e += SK_WARPS * 32) {
    const int row = e % ROWS, col = e / ROWS;
    if (col < M && r0 + row < N) y[(size_t)col * N + r0 + row] = from_f32<OutT>(red[col][row]);
  }
}

template <int NT, int MT, typename OutT>
static int launch(const void* x, const void* W, void* y, int M, int N, int K, cudaStream_t s) {
  const int rows = 16 * MT;
  skinny_kernel<NT, MT, OutT><<<(N + rows - 1) / rows, SK_WARPS * 32, 0, s>>>(
      (const bf16*)x, (const bf16*)W, (OutT*)y, M, N, K);
  return gb_status();
}

template <typename OutT>
static int dispatch(const void* x, const void* W, void* y, int M, int N, int K, cudaStream_t s) {
  if (M <= 8) return launch<1, 1, OutT>(x, W, y, M, N, K, s);
  if (M <= 16) return launch<2, 1, OutT>(x, W, y, M, N, K, s);
  if (M <= 32) return launch<4, 2, OutT>(x, W, y, M, N, K, s);
  return launch<8, 2, OutT>(x, W, y, M, N, K, s);
}

// out_f32: 1 writes 32-bit outputs (logits), 0 writes bf16.
GB_EXPORT int gb_gemm_skinny_bf16(const void* x, const void* W, void* y, int M, int N, int K,
                                  int out_f32, cudaStream_t s) {
  if (M < 0 || N <= 0 || K <= 0) return GB_ERR_BAD_ARG;
  if (M > 64) return GB_ERR_UNSUPPORTED;
  if (K % 8) return GB_ERR_UNSUPPORTED;  // rows must start on 16-byte boundaries
  if ((((uintptr_t)x) | ((uintptr_t)W)) & 15) return GB_ERR_BAD_ARG;
  if (M == 0) return 0;
  return out_f32 ? dispatch<float>(x, W, y, M, N, K, s) : dispatch<bf16>(x, W, y, M, N, K, s);
}
