// True 32-bit matrix product C[M, N] = A[M, K] . W[N, K]^T on the CUDA cores
// (FFMA only: no tensor cores, no TF32), the linear layer of the 32-bit path.
// Weights are row-major [out, in] and activations [tokens, in], as in the
// reference (src/cublas.rs:287-307 does the same product through cuBLAS).
//
// Every output element is summed over k = 0..K-1 in one fixed order, whatever M
// and N are, so a row's result does not depend on how many other rows the step
// holds.  The order is a sum of sums: fused multiply-adds over 32 consecutive k,
// 32 such sums added in turn, and those sums (of 1,024 terms each) added in
// turn.  One chain over all of K would let the rounding error grow with
// sqrt(K): at K = 25,600 (the down projection of the widest model) that showed
// as 5e-5 on logits of order one, beyond the bar the 32-bit path is held to; in
// three levels the longest chain has 32 links.
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16
#define SUM_K 32     // terms of one fused-multiply-add chain
#define SUM_MID 32   // chains added up before their sum is handed on

__global__ void __launch_bounds__(256)
sgemm_nt_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C,
                int M, int N, int K, int lda, int ldw, int ldc) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, 4 x 4 outputs each
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4], mid[4][4], total[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = mid[i][j] = total[i][j] = 0.f;

  // each thread loads 4 elements of A and of W per k-tile: row = tid / 4 (+0),
  // k = (tid % 4) * 4 .. +3
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = k0 + lk + u;
      const int am = m0 + lr, wn = n0 + lr;
      As[lk + u][lr] = (am < M && k < K) ? A[(size_t)am * lda + k] : 0.f;
      Ws[lk + u][lr] = (wn < N && k < K) ? W[(size_t)wn * ldw + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
    const int tile = k0 / BK + 1;
    if (tile % (SUM_K / BK) == 0) {             // 32 terms are in: hand them up
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mid[i][j] += acc[i][j], acc[i][j] = 0.f;
      if (tile % (SUM_K / BK * SUM_MID) == 0) {  // 32 sums of 32 are in: hand them up
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) total[i][j] += mid[i][j], mid[i][j] = 0.f;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)m * ldc + n] = total[i][j] + (mid[i][j] + acc[i][j]);
    }
  }
}

GB_EXPORT int gb_gemm_nt_f32(const float* A, const float* W, float* C, int M, int N, int K, int lda,
                             int ldw, int ldc, cudaStream_t stream) {
  if (M < 0 || N <= 0 || K <= 0 || lda < K || ldw < K || ldc < N) return GB_ERR_BAD_ARG;
  if (M == 0) return 0;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return GB_ERR_UNSUPPORTED;
  sgemm_nt_kernel<<<grid, 256, 0, stream>>>(A, W, C, M, N, K, lda, ldw, ldc);
  return gb_status();
}
