// bf16 matrix product for many rows (a prompt) on pairs of SMs: C = X W^T with
// tcgen05.mma.cta_group::2.
//
// Two thread blocks of a cluster share one 256 x BN tile of C (BN 256, or a
// smaller multiple of 16 on request: see pick_bn).  Block r of the pair loads rows [128 r, 128 r + 128) of the
// tile's X rows and half of its BN rows of W (TMA, 128-byte swizzle, K in steps
// of 64, a ring of six stages of up to 32 KB); one lane of block 0 issues
// M 256 x N BN x K 16 instructions that read the A
// operand's two halves and the B operand's two halves from the shared memory of
// both blocks and accumulate rows 0-127 of the tile in block 0's tensor memory
// and rows 128-255 in block 1's.  Against one block per tile this halves the
// bytes of W that an SM fetches per product, which is what bounds the
// single-block kernel of gemm_tc.cu at these sizes (94 bytes a cycle and SM).
// Accumulators are double-buffered (2 x 256 columns), so the epilogue warps of
// both blocks (TMEM -> registers -> bf16 -> global, optionally silu(gate) * up
// on columns interleaved in eights) drain one tile while the next is multiplied.
//
// Hand-offs: both blocks' loads complete on block 0's `full` barrier (the
// cta_group::2 form of the copy takes a barrier of the pair's first block);
// tcgen05.commit with a cluster mask releases a stage in both blocks and tells
// both blocks' epilogues that a tile is complete; the epilogue warps of both
// blocks arrive on block 0's `acc_empty`.  Tiles go to the clusters round robin,
// X tiles fastest, so that the clusters running together read the same rows of W.
// (The reference calls cuBLAS here, src/cublas.rs:287-307.)
//
// No copy in this file is a multicast copy.  All waits are bounded (tc_common.cuh);
// on expiry a block records a code in args.error and leaves; its partner's waits
// run out the same way.
#include "tc_common.cuh"

#define T2_BM 128      // rows of X per block (256 per pair)
#define T2_BNH 128     // rows of W per block (256 per pair)
#define T2_BN 256
#define T2_BK 64
#ifndef T2_STAGES
#define T2_STAGES 6
#endif
#define T2_THREADS 192  // warp 0: loads; warp 1: MMA issue (first block of the pair); warps 2-5: epilogue

#define GB_ERR_T2_FULL 121
#define GB_ERR_T2_EMPTY 122
#define GB_ERR_T2_ACC_FULL 123
#define GB_ERR_T2_ACC_EMPTY 124

struct Tc2Args {
  void* out;     // [M, ld]
  int* error;    // device int, 0 while all is well
  int M, N, K, ld;
  int out_f32;
  int silu;      // columns of W^T are gate|up interleaved in eights; out is [M, N / 2]
  int bn;        // columns of C per tile: a multiple of 16, 32..256 (filled in by the launcher)
};

static constexpr int T2_A_BYTES = T2_BM * T2_BK * 2;
static constexpr int T2_B_BYTES = T2_BNH * T2_BK * 2;
static constexpr int T2_STAGE_BYTES = T2_A_BYTES + T2_B_BYTES;
static constexpr size_t T2_SMEM = (size_t)T2_STAGES * T2_STAGE_BYTES + 1024 + 256;
// f32 accumulate, bf16 x bf16, both K-major, M = 256 (over the pair); N is added at run time
static constexpr uint32_t T2_IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 4) << 24);

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same variable in block `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_rank(const void* p, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(p)), "r"(rank));
  return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// A tile copy of one block of a pair whose bytes are counted on a barrier of the pair's first block
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
      "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives (once the MMAs issued so far are complete) on the barrier at this
// offset in both blocks of the pair.
__device__ __forceinline__ void tc_commit_pair(void* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"((uint16_t)3)
      : "memory");
}

__device__ __forceinline__ float t2_silu(float g) { return g / (1.0f + __expf(-g)); }

__global__ void __launch_bounds__(T2_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                const Tc2Args a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(tiles + (size_t)T2_STAGES * T2_STAGE_BYTES);
  uint64_t* full = bars;                      // [stages]  used in the pair's first block
  uint64_t* empty = full + T2_STAGES;         // [stages]  in both blocks
  uint64_t* acc_full = empty + T2_STAGES;     // [2]       in both blocks
  uint64_t* acc_empty = acc_full + 2;         // [2]       used in the pair's first block
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  volatile int* abort_flag = &abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int cluster = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const int bn = a.bn, bnh = a.bn / 2;
  const uint32_t stage_tx = T2_A_BYTES + bnh * 128;   // bytes one block loads per stage
  const int tiles_m = (a.M + 255) / 256, tiles_n = (a.N + bn - 1) / bn;
  const int n_tiles = tiles_m * tiles_n;
  const int kblocks = (a.K + T2_BK - 1) / T2_BK;

  if (threadIdx.x == 0) {
    tma_prefetch_map(&map_x);
    tma_prefetch_map(&map_w);
    for (int s = 0; s < T2_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 8);   // four epilogue warps in each block of the pair
    }
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // the same warp in both blocks, as the pair's allocation asks
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&tmem_base_s)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  cluster_sync_all();   // barriers and tensor memory of both blocks exist from here on
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ loads (both blocks)
    if (lane == 0) {
      bool ok = true;
      int s = 0;            // stage and round are kept by counting: this lane's every
      uint32_t round = 0;   // instruction is on the path of the loads
      for (int tile = cluster; tile < n_tiles && ok; tile += n_clusters) {
        const int tm = tile % tiles_m, tn = tile / tiles_m;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&empty[s], (round & 1) ^ 1, abort_flag)) {
            if (!*abort_flag) atomicCAS(a.error, 0, GB_ERR_T2_EMPTY);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t bar = map_to_rank(&full[s], 0);
          if (rank == 0) mbar_expect_tx(&full[s], 2 * stage_tx);   // both blocks' bytes
          uint8_t* sa = tiles + (size_t)s * T2_STAGE_BYTES;
          tma_load_2d_pair(sa, &map_x, kb * T2_BK, tm * 256 + (int)rank * T2_BM, bar);
          tma_load_2d_pair(sa + T2_A_BYTES, &map_w, kb * T2_BK, tn * bn + (int)rank * bnh, bar);
          if (++s == T2_STAGES) {
            s = 0;
            ++round;
          }
        }
      }
      pdl_launch_dependents();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue (first block)
    if (rank == 0 && lane == 0) {
      int s = 0;
      uint32_t round = 0;
      int t = 0;
      bool ok = true;
      const uint32_t idesc = T2_IDESC | ((uint32_t)(bn >> 3) << 17);
      for (int tile = cluster; tile < n_tiles && ok; tile += n_clusters, ++t) {
        const int ab = t & 1;
        if (!mbar_wait(&acc_empty[ab], (((uint32_t)t >> 1) & 1) ^ 1, abort_flag)) {
          if (!*abort_flag) atomicCAS(a.error, 0, GB_ERR_T2_ACC_EMPTY);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t acc = tmem_base + ab * T2_BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&full[s], round & 1, abort_flag)) {
            if (!*abort_flag) atomicCAS(a.error, 0, GB_ERR_T2_FULL);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + (size_t)s * T2_STAGE_BYTES);
          const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + T2_A_BYTES);
#pragma unroll
          for (int k = 0; k < T2_BK / 16; ++k)
            tc_mma_pair(acc, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit_pair(&empty[s]);      // the stage is free in both blocks
          if (++s == T2_STAGES) {
            s = 0;
            ++round;
          }
        }
        if (ok) tc_commit_pair(&acc_full[ab]);   // both blocks may drain their half of the tile
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both blocks)
    const int q = warp & 3;   // the TMEM lanes this warp may touch
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const int n_out = a.silu ? a.N / 2 : a.N;
    int t = 0;
    bool ok = true;
    for (int tile = cluster; tile < n_tiles && ok; tile += n_clusters, ++t) {
      const int tm = tile % tiles_m, tn = tile / tiles_m;
      const int ab = t & 1;
      if (!mbar_wait_warp(&acc_full[ab], ((uint32_t)t >> 1) & 1, abort_flag)) {
        if (lane == 0) {
          if (!*abort_flag) atomicCAS(a.error, 0, GB_ERR_T2_ACC_FULL);
          *abort_flag = 1;
        }
        break;
      }
      tc_fence_after();
      const int row = tm * 256 + (int)rank * T2_BM + q * 32 + lane;
      const int col0 = tn * bn;
#pragma unroll 1
      for (int c0 = 0; c0 < bn; c0 += 16) {   // 16 columns: 32 bytes of a bf16 row, or one gate|up group
        uint32_t v[16];
        tc_ld16(lane_addr + ab * T2_BN + c0, v);
        tc_wait_ld();
        const int col = col0 + c0;
        if (row >= a.M || col >= a.N) continue;
        if (a.silu) {
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float g0 = __uint_as_float(v[2 * i]), g1 = __uint_as_float(v[2 * i + 1]);
            const float u0 = __uint_as_float(v[8 + 2 * i]), u1 = __uint_as_float(v[8 + 2 * i + 1]);
            w[i] = pack2(t2_silu(g0) * u0, t2_silu(g1) * u1);
          }
          *reinterpret_cast<uint4*>((bf16*)a.out + (size_t)row * a.ld + col / 2) = make_uint4(w[0], w[1], w[2], w[3]);
        } else if (a.out_f32) {
          float* orow = (float*)a.out + (size_t)row * a.ld + col;
#pragma unroll
          for (int c = 0; c < 16; c += 4) {
            if (col + c + 3 < n_out) {
              *reinterpret_cast<float4*>(orow + c) = make_float4(__uint_as_float(v[c]), __uint_as_float(v[c + 1]),
                                                                  __uint_as_float(v[c + 2]), __uint_as_float(v[c + 3]));
            } else {
              for (int e = 0; e < 4; ++e)
                if (col + c + e < n_out) orow[c + e] = __uint_as_float(v[c + e]);
            }
          }
        } else {
          bf16* orow = (bf16*)a.out + (size_t)row * a.ld + col;
#pragma unroll
          for (int c = 0; c < 16; c += 8) {
            if (col + c + 7 < n_out) {
              uint4 w;
              w.x = pack2(__uint_as_float(v[c]), __uint_as_float(v[c + 1]));
              w.y = pack2(__uint_as_float(v[c + 2]), __uint_as_float(v[c + 3]));
              w.z = pack2(__uint_as_float(v[c + 4]), __uint_as_float(v[c + 5]));
              w.w = pack2(__uint_as_float(v[c + 6]), __uint_as_float(v[c + 7]));
              *reinterpret_cast<uint4*>(orow + c) = w;
            } else {
              for (int e = 0; e < 8; ++e)
                if (col + c + e < n_out) orow[c + e] = __float2bfloat16(__uint_as_float(v[c + e]));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_rank(&acc_empty[ab], 0));   // the accumulator may be reused
    }
    (void)ok;
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  cluster_sync_all();   // neither block leaves while its partner may still touch its memory
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u)
                 : "memory");
  }
}

// X [M, K] and W [N, K] bf16, row pitch K, 16-byte aligned; out [M, ld] bf16 or
// float (ld = N, or N / 2 with silu).  K % 8 == 0 (a row pitch must be a multiple
// of 16 bytes for TMA); with silu N % 16 == 0; ld and the output pointer must
// allow 16-byte stores.
// Columns per tile: 256 unless the caller says otherwise.  Narrower tiles that
// would fill the last round of tiles better were measured and do not pay: an
// instruction over the pair takes about 120 cycles however few columns it has
// (2,048 x 2,560 x 4,096: 50.5 us with every width from 144 to 256, 71 us with
// 128), so a k-block costs the same and only the wide tile uses it fully.
static int pick_bn(int, int, int) { return T2_BN; }

GB_EXPORT int gb_gemm_tc2_bf16(const void* X, const void* W, const Tc2Args* args, cudaStream_t s) {
  Tc2Args a = *args;
  if (!X || !W || !a.out || !a.error || a.M <= 0 || a.N <= 0 || a.K <= 0) return GB_ERR_BAD_ARG;
  if (a.K % 8) return GB_ERR_UNSUPPORTED;
  if ((((uintptr_t)X) | ((uintptr_t)W) | ((uintptr_t)a.out)) & 15) return GB_ERR_BAD_ARG;
  if (a.silu && (a.N % 16 || a.out_f32)) return GB_ERR_UNSUPPORTED;
  if ((a.ld * (a.out_f32 ? 4 : 2)) % 16) return GB_ERR_UNSUPPORTED;
  static int sms = 0;
  static bool configured = false;
  if (!configured) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemm_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)T2_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap mx, mw;
  int e = tc_make_map_2d(&mx, X, (uint64_t)a.M, (uint64_t)a.K, (uint64_t)a.K * 2, T2_BM, T2_BK);
  if (e) return e;
  if (a.bn <= 0) a.bn = pick_bn(a.M, a.N, sms / 2);
  if (a.bn % 16 || a.bn < 32 || a.bn > T2_BN) return GB_ERR_BAD_ARG;
  e = tc_make_map_2d(&mw, W, (uint64_t)a.N, (uint64_t)a.K, (uint64_t)a.K * 2, a.bn / 2, T2_BK);
  if (e) return e;
  const long long n_tiles = (long long)((a.M + 255) / 256) * ((a.N + a.bn - 1) / a.bn);
  long long clusters = sms / 2;
  if (clusters > n_tiles) clusters = n_tiles;
  if (clusters < 1) return GB_ERR_UNSUPPORTED;
  return gb_launch_cluster(gemm_tc2_kernel, dim3((unsigned)(2 * clusters)), dim3(T2_THREADS), T2_SMEM, s, 2,
                           mx, mw, a);
}
