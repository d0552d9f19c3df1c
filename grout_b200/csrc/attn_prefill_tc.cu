// Causal attention of prompt tokens over the paged cache on the fifth-generation
// tensor cores: both products of flash attention are tcgen05.mma with their
// results in tensor memory.  (The reference's prefill kernels are cuTile tile
// programs, src/kernels.rs:1146-1295, 1513-1862; its online-softmax recurrence
// in the log2 domain is the one used here.)
//
// One block owns 128 consecutive query rows of one sequence and one query head.
// Key tiles are whole pages (64 keys).  Per key tile j:
//   S_j  = Q K_j^T          tcgen05.mma, M 128 x N 64 x K head_dim, Q and K_j
//                           K-major tiles that TMA wrote (128-byte swizzle)
//   P_j  = 2^(S_j c - m_j)  softmax threads (one per query row) read S_j from
//                           TMEM, mask, keep the row maximum m and sum l, and
//                           write P_j as bf16 into shared memory in the same
//                           swizzled K-major layout
//   R_j  = P_j V_j          tcgen05.mma, M 128 x N head_dim x K 64, V_j read as
//                           an MN-major operand straight from the page layout
//   O    = O 2^(m_{j-1}-m_j) + R_j   in registers, one row per thread
// S and R are double-buffered in TMEM (2 x 64 + 2 x head_dim columns), the K/V
// ring has three stages, so the tensor cores work on tile j + 1 while tile j is
// in the softmax.
//
// Warps: 0 = TMA producer (one lane), 1 = TMEM allocation and MMA issue (one
// lane), 2-9 = softmax / accumulation / store: two threads per query row, each
// with half of a tile's keys and half of head_dim, so that every scheduler of the
// SM holds two such warps.
//
// Pages must hold finite values in rows beyond a sequence's length (the cache is
// zero-filled when it is made): those keys are masked to probability 0, and
// 0 x NaN would still be NaN in the second product.
// All mbarrier waits are bounded (see tc_common.cuh); on expiry the block sets
// args.error, stops, frees its tensor memory and returns.
#include "tc_common.cuh"

#define AT_BM 128
#define AT_BN 64
#define AT_THREADS 320
#define AT_STAGES 3

#define GB_ERR_AT_TIMEOUT 111

struct AttnTcArgs {
  const int* block_table;  // [slots, max_pages]
  const int* cu_q;         // [n_seqs + 1]
  const int* slots;        // [n_seqs]
  const int* kv_len;       // [n_seqs]
  bf16* out;               // [n_tokens, nq, D]
  int* error;
  int n_seqs, nq, nkv, max_pages, window, n_qblocks;
  float scale_log2;
};

// V tile as the B operand of R = P V: N (head_dim) is the contiguous direction
// ("MN-major").  In the tile that TMA wrote, a key is a 128-byte row holding 64
// head_dim elements: 8-key groups are 1024 bytes apart (stride byte offset) and
// the next 64 elements of head_dim are a whole sub-tile further (leading byte
// offset).
__device__ __forceinline__ uint64_t make_smem_desc_mn(uint32_t saddr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ float fast_exp2(float x) {   // 2^x, one MUFU operation; 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int DS>   // head_dim = 64 * DS
struct AtConfig {
  static constexpr int D = 64 * DS;
  static constexpr int Q_BYTES = AT_BM * 128 * DS;          // DS sub-tiles of [128][64]
  static constexpr int SUB_BYTES = AT_BN * 128;             // one [64 keys][64] sub-tile
  static constexpr int KV_BYTES = 2 * DS * SUB_BYTES;       // K and V of one stage
  static constexpr int P_BYTES = AT_BM * 128;               // [128][64 keys]
  static constexpr int TMEM_S = 0;                          // two S buffers of 64 columns
  static constexpr int TMEM_R = 2 * AT_BN;                  // two R buffers of D columns
  static constexpr int TMEM_COLS = (2 * AT_BN + 2 * D) <= 256 ? 256 : 512;
  static constexpr size_t SMEM = (size_t)Q_BYTES + AT_STAGES * KV_BYTES + 2 * P_BYTES + 1024 + 256;
  // S = Q K^T: both K-major, N = 64.   R = P V: A K-major, B MN-major (bit 16), N = D.
  static constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(AT_BN >> 3) << 17) |
                                      ((uint32_t)(AT_BM >> 4) << 24);
  static constexpr uint32_t IDESC_R = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                                      ((uint32_t)(D >> 3) << 17) | ((uint32_t)(AT_BM >> 4) << 24);
};

template <int DS>
__global__ void __launch_bounds__(AT_THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const AttnTcArgs a) {
  using Cfg = AtConfig<DS>;
  constexpr int D = Cfg::D;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* q_s = base;
  uint8_t* kv_s = q_s + Cfg::Q_BYTES;                       // [stage][K sub-tiles | V sub-tiles]
  uint8_t* p_s = kv_s + AT_STAGES * Cfg::KV_BYTES;          // [2][P_BYTES]
  uint64_t* bars = (uint64_t*)(p_s + 2 * Cfg::P_BYTES);
  uint64_t* q_full = bars;                 // 1
  uint64_t* kv_full = bars + 1;            // [3]
  uint64_t* kv_empty = kv_full + AT_STAGES;
  uint64_t* s_full = kv_empty + AT_STAGES; // [2]
  uint64_t* s_empty = s_full + 2;
  uint64_t* p_full = s_empty + 2;
  uint64_t* p_empty = p_full + 2;
  uint64_t* r_full = p_empty + 2;
  uint64_t* r_empty = r_full + 2;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ float xch[6 * AT_BM];   // halves of row maxima (2 tiles x 2 groups) and of l
  volatile int* abort_flag = &abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y;
  const int qb = a.n_qblocks - 1 - blockIdx.x;   // heavy blocks first

  // which sequence does this query block belong to?
  int seq = 0, first_block = 0, q_len = 0;
  for (; seq < a.n_seqs; ++seq) {
    q_len = a.cu_q[seq + 1] - a.cu_q[seq];
    const int nb = (q_len + AT_BM - 1) / AT_BM;
    if (qb < first_block + nb) break;
    first_block += nb;
  }
  if (seq >= a.n_seqs) return;
  const int q0 = (qb - first_block) * AT_BM;
  const int rows = min(AT_BM, q_len - q0);
  const int tok0 = a.cu_q[seq] + q0;
  const int slot = a.slots[seq];
  const size_t tok_stride = (size_t)a.nq * D;
  if (slot < 0) {   // padding sequence: zeros
    bf16* out = a.out + ((size_t)tok0 * a.nq + h) * D;
    for (int i = threadIdx.x; i < rows * D; i += AT_THREADS)
      out[(size_t)(i / D) * tok_stride + (i % D)] = __float2bfloat16(0.f);
    return;
  }
  const int kv_len = a.kv_len[seq];
  const int pos0 = kv_len - q_len + q0;
  const int kvh = h / (a.nq / a.nkv);
  const int* table = a.block_table + (size_t)slot * a.max_pages;
  const int key_hi = pos0 + rows - 1;
  const int key_lo = (a.window > 0 && pos0 - a.window + 1 > 0) ? pos0 - a.window + 1 : 0;
  const int tile_lo = key_lo / AT_BN, n_tiles = key_hi / AT_BN - tile_lo + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < AT_STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 8);   // one arrival per softmax warp
      mbar_init(&p_full[i], 8);
      mbar_init(&p_empty[i], 1);
      mbar_init(&r_full[i], 1);
      mbar_init(&r_empty[i], 8);
    }
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&tmem_base_s)),
                 "r"((uint32_t)Cfg::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      mbar_expect_tx(q_full, Cfg::Q_BYTES);
      for (int ds = 0; ds < DS; ++ds)
        tma_load_2d(q_s + ds * (AT_BM * 128), &map_q, h * D + ds * 64, tok0, q_full);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % AT_STAGES;
        if (!mbar_wait(&kv_empty[s], (((uint32_t)(j / AT_STAGES)) & 1) ^ 1, abort_flag)) {
          if (!*abort_flag) atomicCAS(a.error, 0, GB_ERR_AT_TIMEOUT);
          *abort_flag = 1;
          break;
        }
        const int page = table[tile_lo + j];
        const int row0 = (page * a.nkv + kvh) * AT_BN;
        uint8_t* st = kv_s + (size_t)s * Cfg::KV_BYTES;
        mbar_expect_tx(&kv_full[s], Cfg::KV_BYTES);
        for (int ds = 0; ds < DS; ++ds) {
          tma_load_2d(st + ds * Cfg::SUB_BYTES, &map_k, ds * 64, row0, &kv_full[s]);
          tma_load_2d(st + (DS + ds) * Cfg::SUB_BYTES, &map_v, ds * 64, row0, &kv_full[s]);
        }
      }
      pdl_launch_dependents();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0, abort_flag);
      auto issue_r = [&](int i) -> bool {   // R_i = P_i V_i
        const int b = i & 1, s = i % AT_STAGES;
        if (!mbar_wait(&p_full[b], ((uint32_t)(i >> 1)) & 1, abort_flag)) return false;
        if (!mbar_wait(&r_empty[b], (((uint32_t)(i >> 1)) & 1) ^ 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t pa = smem_u32(p_s + b * Cfg::P_BYTES);
        const uint32_t va = smem_u32(kv_s + (size_t)s * Cfg::KV_BYTES + DS * Cfg::SUB_BYTES);
        const uint64_t dp = make_smem_desc(pa);
        const uint64_t dv = make_smem_desc_mn(va, Cfg::SUB_BYTES);
        const uint32_t tr = tmem_base + Cfg::TMEM_R + b * D;
#pragma unroll
        for (int k = 0; k < AT_BN / 16; ++k)   // 16 keys: 32 bytes of a P row, 2 key groups of V
          tc_mma(tr, dp + 2 * k, dv + (uint64_t)((2 * 1024) >> 4) * k, Cfg::IDESC_R, k > 0 ? 1u : 0u);
        tc_commit(&r_full[b]);
        tc_commit(&kv_empty[s]);   // K_i was read by S_i, V_i by R_i: the stage is free
        tc_commit(&p_empty[b]);
        return true;
      };
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int b = j & 1, s = j % AT_STAGES;
        ok = mbar_wait(&kv_full[s], ((uint32_t)(j / AT_STAGES)) & 1, abort_flag) &&
             mbar_wait(&s_empty[b], (((uint32_t)(j >> 1)) & 1) ^ 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t qa = smem_u32(q_s);
        const uint32_t ka = smem_u32(kv_s + (size_t)s * Cfg::KV_BYTES);
        const uint32_t ts = tmem_base + Cfg::TMEM_S + b * AT_BN;
#pragma unroll
        for (int ds = 0; ds < DS; ++ds) {
          const uint64_t dq = make_smem_desc(qa + ds * (AT_BM * 128));
          const uint64_t dk = make_smem_desc(ka + ds * Cfg::SUB_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma(ts, dq + 2 * k, dk + 2 * k, Cfg::IDESC_S, (ds > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(&s_full[b]);
        if (j >= 1) ok = issue_r(j - 1);
      }
      if (ok) ok = issue_r(n_tiles - 1);
      if (!ok) {
        if (!*abort_flag) atomicCAS(a.error, 0, GB_ERR_AT_TIMEOUT);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax, accumulate, store
    // Two threads share a query row: group 0 (warps 2-5) owns key columns 0-31 of
    // every tile and the first half of head_dim, group 1 (warps 6-9) the rest.  The
    // halves of a row's maximum meet in shared memory once per tile.
    constexpr int HC = AT_BN / 2, HD = D / 2;
    const int grp = (warp - 2) >> 2;
    const int q = warp & 3;                        // the TMEM lanes this warp may read
    const int r = q * 32 + lane;                   // query row of the block
    const int pos = pos0 + r;
    const int hi = r < rows ? pos : -1;            // rows beyond the block see nothing
    const int lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    float o[HD];
#pragma unroll
    for (int d = 0; d < HD; ++d) o[d] = 0.f;
    float m = -INFINITY, l = 0.f, corr_prev = 0.f;
    bool ok = true;

    auto wait_warp = [&](uint64_t* bar, uint32_t parity) -> bool {
      int got = 0;
      if (lane == 0) got = mbar_wait(bar, parity, nullptr) ? 1 : 0;
      return __shfl_sync(0xffffffffu, got, 0) != 0;
    };
    auto accumulate = [&](int i, float corr) -> bool {   // O = O corr + R_i, this group's half
      const int b = i & 1;
      if (!wait_warp(&r_full[b], ((uint32_t)(i >> 1)) & 1)) return false;
      tc_fence_after();
      uint32_t v[HD];
      if constexpr (HD == 64) tc_ld64(lane_addr + Cfg::TMEM_R + b * D + grp * HD, v);
      else tc_ld32(lane_addr + Cfg::TMEM_R + b * D + grp * HD, v);
      tc_wait_ld();
#pragma unroll
      for (int j = 0; j < HD; ++j) o[j] = o[j] * corr + __uint_as_float(v[j]);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&r_empty[b]);
      return true;
    };

    for (int j = 0; j < n_tiles && ok; ++j) {
      const int b = j & 1;
      if (!wait_warp(&s_full[b], ((uint32_t)(j >> 1)) & 1)) { ok = false; break; }
      tc_fence_after();
      float s[HC];
      {
        uint32_t v[HC];
        tc_ld32(lane_addr + Cfg::TMEM_S + b * AT_BN + grp * HC, v);
        tc_wait_ld();
#pragma unroll
        for (int jj = 0; jj < HC; ++jj) s[jj] = __uint_as_float(v[jj]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[b]);   // S_j is in registers: the buffer is free

      const int key0 = (tile_lo + j) * AT_BN + grp * HC;
      // a tile that lies wholly at or below the block's first position (and inside
      // every row's window) needs no mask
      const bool need_mask = (tile_lo + j) * AT_BN + AT_BN - 1 > pos0 || a.window > 0 || rows < AT_BM;
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < HC; ++c) {
          const int key = key0 + c;
          if (key < lo || key > hi) s[c] = -INFINITY;
        }
      }
      // row maximum of the raw scores (the scale is positive), four chains
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < HC; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], s[c]);
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      xch[(b * 2 + grp) * AT_BM + r] = mx;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      mx = fmaxf(mx, xch[(b * 2 + (grp ^ 1)) * AT_BM + r]) * a.scale_log2;
      const float m_new = fmaxf(m, mx);
      const float mbase = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = (m == -INFINITY) ? 0.f : fast_exp2(m - mbase);
      m = m_new;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[HC / 2];
#pragma unroll
      for (int c = 0; c < HC; c += 2) {
        const float e0 = fast_exp2(fmaf(s[c], a.scale_log2, -mbase));
        const float e1 = fast_exp2(fmaf(s[c + 1], a.scale_log2, -mbase));
        sum4[(c >> 1) & 3] += e0 + e1;
        pk[c / 2] = pack2(e0, e1);
      }
      l = l * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));   // this group's share of l

      // P_j into shared memory, K-major [128 rows][64 keys] under the 128-byte swizzle
      if (!wait_warp(&p_empty[b], (((uint32_t)(j >> 1)) & 1) ^ 1)) { ok = false; break; }
      {
        uint8_t* prow = p_s + b * Cfg::P_BYTES + r * 128;
#pragma unroll
        for (int c4 = 0; c4 < HC / 8; ++c4) {
          const int ch = grp * (HC / 8) + c4;
          const uint4 w = make_uint4(pk[4 * c4], pk[4 * c4 + 1], pk[4 * c4 + 2], pk[4 * c4 + 3]);
          *reinterpret_cast<uint4*>(prow + ((ch ^ (r & 7)) << 4)) = w;
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[b]);

      if (j >= 1) ok = accumulate(j - 1, corr_prev);
      corr_prev = corr;
    }
    if (ok) ok = accumulate(n_tiles - 1, corr_prev);
    if (!ok) {
      if (lane == 0) {
        atomicCAS(a.error, 0, GB_ERR_AT_TIMEOUT);
        *abort_flag = 1;
      }
    } else {
      // the two halves of l meet, then each group stores its half of the row
      xch[(4 + grp) * AT_BM + r] = l;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      const float inv = 1.0f / (l + xch[(4 + (grp ^ 1)) * AT_BM + r]);
      if (r < rows) {
        bf16* orow = a.out + ((size_t)(tok0 + r) * a.nq + h) * D + grp * HD;
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 8) {
          uint4 w;
          w.x = pack2(o[c0] * inv, o[c0 + 1] * inv);
          w.y = pack2(o[c0 + 2] * inv, o[c0 + 3] * inv);
          w.z = pack2(o[c0 + 4] * inv, o[c0 + 5] * inv);
          w.w = pack2(o[c0 + 6] * inv, o[c0 + 7] * inv);
          *reinterpret_cast<uint4*>(orow + c0) = w;
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)Cfg::TMEM_COLS)
                 : "memory");
  }
}

template <int DS>
static int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                  const AttnTcArgs& a, cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<DS>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)AtConfig<DS>::SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return gb_launch(attn_prefill_tc_kernel<DS>, dim3(a.n_qblocks, a.nq), dim3(AT_THREADS),
                   AtConfig<DS>::SMEM, s, mq, mk, mv, a);
}

// q [n_tokens, nq, D]; k_pages and v_pages [n_pages, nkv, 64, D]; bf16.
// head_dim 64 or 128 and pages of 64 tokens; anything else is refused
// (GB_ERR_UNSUPPORTED) and the caller uses another kernel.
GB_EXPORT int gb_attn_prefill_tc(const void* q, const void* k_pages, const void* v_pages,
                                 const AttnTcArgs* a, int n_tokens, long long n_pages, int D, int page,
                                 cudaStream_t s) {
  if (!q || !k_pages || !v_pages || !a->out || !a->error || a->n_seqs <= 0 || a->nq <= 0 ||
      a->nkv <= 0 || a->nq % a->nkv || a->max_pages <= 0 || a->n_qblocks < 0 || n_tokens <= 0 ||
      n_pages <= 0)
    return GB_ERR_BAD_ARG;
  if (page != AT_BN || (D != 64 && D != 128) || a->nq > 65535) return GB_ERR_UNSUPPORTED;
  if (n_pages * a->nkv * AT_BN > 0x7fffffffll) return GB_ERR_UNSUPPORTED;
  if (a->n_qblocks == 0) return 0;
  CUtensorMap mq, mk, mv;
  int e = tc_make_map_2d(&mq, q, (uint64_t)n_tokens, (uint64_t)a->nq * D, (uint64_t)a->nq * D * 2,
                         AT_BM, 64);
  if (e) return e;
  const uint64_t kv_rows = (uint64_t)n_pages * a->nkv * AT_BN;
  e = tc_make_map_2d(&mk, k_pages, kv_rows, (uint64_t)D, (uint64_t)D * 2, AT_BN, 64);
  if (e) return e;
  e = tc_make_map_2d(&mv, v_pages, kv_rows, (uint64_t)D, (uint64_t)D * 2, AT_BN, 64);
  if (e) return e;
  return D == 64 ? launch<1>(mq, mk, mv, *a, s) : launch<2>(mq, mk, mv, *a, s);
}
