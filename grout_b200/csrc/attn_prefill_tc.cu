// Causal attention of prompt tokens over the paged cache on the fifth-generation
// tensor cores: both products of flash attention are tcgen05.mma with their
// results in tensor memory.  (The reference's prefill kernels are cuTile tile
// programs, src/kernels.rs:1146-1295, 1513-1862; its online-softmax recurrence
// in the log2 domain is the one used here.)
//
// One block owns 256 consecutive query rows of one sequence and one query head,
// as two query blocks A and B of 128 rows that share every key tile.  Key tiles
// are whole pages (64 keys).  Per key tile j and query block g:
//   S_gj = Q_g K_j^T        tcgen05.mma, M 128 x N 64 x K head_dim; Q_g lives in
//                           tensor memory for the whole block (the softmax threads
//                           put their own query row there once), K_j is a K-major
//                           tile that TMA wrote (128-byte swizzle)
//   P_gj = 2^(S_gj c - b)   softmax threads (one per query row) read S_gj from
//                           TMEM, mask, and write P_gj as bf16 into shared memory
//                           in the swizzled K-major layout
//   O_g += P_gj V_j         tcgen05.mma accumulating in TMEM, M 128 x N head_dim
//                           x K 64, V_j read as an MN-major operand straight from
//                           the page layout
// Why Q sits in tensor memory: with one SM per tile the tensor core fetches its
// shared-memory operands at about 64 bytes a cycle (measured: the issue of the
// products, not their arithmetic, set the tile time), and Q was two thirds of
// the bytes of the first product.
// The base b of a row is its running maximum, but it is only raised (and the
// row of O_g in TMEM rescaled) when the maximum has grown by more than 2^8, so
// that the read-modify-write of O is rare; probabilities then stay below 256,
// and the final division by l removes the base.
// The two query blocks are two independent chains (barrier, TMEM load, softmax,
// fence, barrier) that overlap each other and the tensor cores; P is double-
// buffered per block, the K/V ring has four stages.
// TMEM columns: Q 2 x head_dim/2, S 2 x 64, O 2 x head_dim.
//
// Warps: 0 = TMA producer (one lane), 1 = TMEM allocation and MMA issue for
// query block A, 10 = MMA issue for block B (the warp walks an event loop, an
// elected lane issues), 2-5 = softmax of block A (thread = query row), 6-9 = of
// block B.  One issuing warp per query block: a single one was the bottleneck
// (its waits, polls and blocking issues in series took longer than a softmax
// tile), and it kept both blocks in lockstep.
//
// Pages must hold finite values in rows beyond a sequence's length (the cache is
// zero-filled when it is made): those keys are masked to probability 0, and
// 0 x NaN would still be NaN in the second product.
// All mbarrier waits are bounded (see tc_common.cuh); on expiry the block sets
// args.error, stops, frees its tensor memory and returns.
// With -DAT_STAMPS the heaviest block of head 0 writes clock stamps behind the
// error word (from 64 ints in; the caller must give it 2.5 KB of room): eight
// per tile for tiles 8-11 of one softmax warp of each query block, then up to 96
// issue events (clock << 20 | tile << 8 | block << 4 | 1 for S, 2 for PV) of
// each issuing warp.  With -DAT_BLOCK_STAMPS instead, every block writes eight
// 64-bit words there (index y * gridDim.x + x): %globaltimer at its start, after
// the wait for the producer kernel, at its first product, after its softmax
// loop, after its epilogue and at its exit, then its number of key tiles and
// its SM: this is how the order in which blocks reach the SMs was seen.
// Tuning aids; never defined in the product build.
#include "tc_common.cuh"

#define AT_BM 128
#define AT_BN 64

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

// The softmax threads are bound by how many instructions they issue as much as by the
// exponentials, so the arithmetic around the exponentials is done two values at a time
// (the packed 32-bit operations of this architecture) and the maximum three at a time.
// An arrival by the lanes for which pred holds, as a predicated instruction: no branch for
// the warp to diverge at and come together after.
__device__ __forceinline__ void mbar_arrive_if(void* bar, bool pred) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %1, 0;\n\t@p mbarrier.arrive.shared::cta.b64 _, [%0];\n\t}" ::"r"(
                   smem_u32(bar)),
               "r"((uint32_t)pred)
               : "memory");
}
// A wait for a thread that is far ahead of what it waits for (the producer, by the depth of
// its ring): it sleeps between polls instead of taking issue slots from the warps that work.
__device__ __forceinline__ bool mbar_wait_idle(void* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try(bar, parity)) return true;
  const unsigned long long t0 = now_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i) {
      __nanosleep(200);
      if (mbar_try(bar, parity)) return true;
    }
    if (*abort_flag) return mbar_try(bar, parity);
    if (now_ns() - t0 > TC_WAIT_LIMIT_NS) return false;
  }
}
__device__ __forceinline__ void sts128(uint32_t saddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
  return v;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {   // a * b + c, both halves
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

template <int DS, int G>   // head_dim = 64 * DS; G query blocks of 128 rows per thread block
struct AtConfig {
  static constexpr int D = 64 * DS;
  // G = 2: one block per SM, four K/V stages.  G = 1: a block of half the size, two of
  // which share an SM (two stages each): finer pieces of work for the SMs to share out
  // when a step has few query rows, and the two blocks overlap like the two query blocks.
  static constexpr int STAGES = G == 2 ? 4 : 2;
  static constexpr int NSW = 4;                             // softmax warps per query block
  static constexpr int MMA_B_WARP = 2 + G * NSW;            // (G = 2 only) the issuing warp of block B
  static constexpr int THREADS = 32 * (2 + G * NSW + (G == 2 ? 1 : 0));
  static constexpr int SUB_BYTES = AT_BN * 128;             // one [64 keys][64] sub-tile
  static constexpr int KV_BYTES = 2 * DS * SUB_BYTES;       // K and V of one stage
  static constexpr int P_BYTES = AT_BM * 128;               // [128][64 keys]; two per query block
  static constexpr int TMEM_Q = 0;                          // Q[g]: D/2 columns each (two bf16 a column)
  static constexpr int TMEM_S = G * 64;                     // S[g]: 64 columns each
  static constexpr int TMEM_O = G * 128;                    // O[g]: D columns each
  static constexpr int TMEM_COLS = G * 256;
  static constexpr size_t SMEM = (size_t)STAGES * KV_BYTES + 2 * G * P_BYTES + 1024 + 256;
  // S = Q K^T: both K-major, N = 64.   O += P V: A K-major, B MN-major (bit 16), N = D.
  static constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(AT_BN >> 3) << 17) |
                                      ((uint32_t)(AT_BM >> 4) << 24);
  static constexpr uint32_t IDESC_R = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                                      ((uint32_t)(D >> 3) << 17) | ((uint32_t)(AT_BM >> 4) << 24);
};

#ifdef AT_STAMPS
#define AT_STAMP(buf, slot) \
  if (stamping && j >= 8 && j < 12) (buf)[slot] = clock64();
#else
#define AT_STAMP(buf, slot)
#endif

template <int DS, int G>
__global__ void __launch_bounds__((AtConfig<DS, G>::THREADS), (G == 2 ? 1 : 2))
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const bf16* q_rows, const AttnTcArgs a) {
  using Cfg = AtConfig<DS, G>;
  constexpr int AT_STAGES = Cfg::STAGES;
  constexpr int D = Cfg::D;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* kv_s = base;                                     // [stage][K sub-tiles | V sub-tiles]
  uint8_t* p_s = kv_s + AT_STAGES * Cfg::KV_BYTES;          // [query block][2 buffers][P_BYTES]
  uint64_t* bars = (uint64_t*)(p_s + 2 * G * Cfg::P_BYTES);
  uint64_t* kv_full = bars;                  // [stages]
  uint64_t* kv_empty = kv_full + AT_STAGES;  // [g][stages]: query block g has read the stage
  uint64_t* q_full = kv_empty + 2 * AT_STAGES;   // [g]: the block's queries are in tensor memory
  uint64_t* s_full = q_full + 2;             // [g]
  uint64_t* s_empty = s_full + 2;            // [g]: the softmax threads hold S in registers
  uint64_t* p_full = s_empty + 2;            // [g][2]
  uint64_t* o_done = p_full + 4;             // [g]: the product of tile j has been added to O_g
  uint64_t* o_final = o_done + 2;            // [g]: the last product has been added to O_g
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  volatile int* abort_flag = &abort_s;

  // (taken from lane 0, so that the compiler knows it is the same in the whole warp)
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
  const int h = blockIdx.x;
#ifdef AT_BLOCK_STAMPS
  unsigned long long* bst = (unsigned long long*)(a.error + 64) + ((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 8;
  if (threadIdx.x == 0) { bst[0] = now_ns(); unsigned sm; asm("mov.u32 %0, %smid;" : "=r"(sm)); bst[7] = sm; }
#define BST(i) bst[i] = now_ns();
#else
#define BST(i)
#endif
  // Blocks are handed to the SMs in the order of their index, x fastest: the heads
  // are x and the query blocks y, last (longest) first, so that every head's heavy
  // blocks start before any light one and the light ones fill the gaps at the end.
  const int qb = a.n_qblocks - 1 - blockIdx.y;

  // which sequence does this pair of query blocks belong to?
  int seq = 0, first_block = 0, q_len = 0;
  for (; seq < a.n_seqs; ++seq) {
    q_len = a.cu_q[seq + 1] - a.cu_q[seq];
    const int nb = (q_len + G * AT_BM - 1) / (G * AT_BM);
    if (qb < first_block + nb) break;
    first_block += nb;
  }
  if (seq >= a.n_seqs) return;
  const int q0 = (qb - first_block) * G * AT_BM;
  const int rows = min(G * AT_BM, q_len - q0);          // rows of the block
  const int tok0 = a.cu_q[seq] + q0;
  const int slot = a.slots[seq];
  const size_t tok_stride = (size_t)a.nq * D;
  if (slot < 0) {   // padding sequence: zeros
    bf16* out = a.out + ((size_t)tok0 * a.nq + h) * D;
    for (int i = threadIdx.x; i < rows * D; i += Cfg::THREADS)
      out[(size_t)(i / D) * tok_stride + (i % D)] = __float2bfloat16(0.f);
    return;
  }
  const int kv_len = a.kv_len[seq];
  const int pos0 = kv_len - q_len + q0;                 // position of the pair's first row
  const int kvh = h / (a.nq / a.nkv);
  const int* table = a.block_table + (size_t)slot * a.max_pages;
  const bool has_b = G == 2 && rows > AT_BM;
  const int rows_a = min(rows, AT_BM), rows_b = rows - AT_BM;
  const int key_lo = (a.window > 0 && pos0 - a.window + 1 > 0) ? pos0 - a.window + 1 : 0;
  const int tile_lo = key_lo / AT_BN;
  // tiles each query block needs (both start at tile_lo; A needs fewer at the end)
  const int n_a = (pos0 + rows_a - 1) / AT_BN - tile_lo + 1;
  const int n_b = has_b ? (pos0 + rows - 1) / AT_BN - tile_lo + 1 : 0;
  const int n_tiles = has_b ? n_b : n_a;
#ifdef AT_STAMPS
  long long* stamp_buf = (long long*)(a.error + 64);
#endif

  if (threadIdx.x == 0) {
    tma_prefetch_map(&map_k);
    tma_prefetch_map(&map_v);
    for (int s = 0; s < AT_STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
      mbar_init(&kv_empty[AT_STAGES + s], 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(&q_full[g], Cfg::NSW);    // one arrival per softmax warp of the group
      mbar_init(&s_full[g], 1);
      mbar_init(&s_empty[g], Cfg::NSW);
      mbar_init(&o_done[g], 1);
      mbar_init(&o_final[g], 1);
    }
    for (int i = 0; i < 4; ++i) {   // (with one query block the second half is unused)
      mbar_init(&p_full[i], Cfg::NSW);
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
  if (threadIdx.x == 0) { BST(1) }

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % AT_STAGES;
        // the tile that held this stage has been read by the query blocks that needed it
        const uint32_t par = (((uint32_t)(j / AT_STAGES)) & 1) ^ 1;
        bool freed = j - AT_STAGES >= n_a || mbar_wait_idle(&kv_empty[s], par, abort_flag);
        freed = freed && (j - AT_STAGES >= n_b || mbar_wait_idle(&kv_empty[AT_STAGES + s], par, abort_flag));
        if (!freed) {
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
  } else if (warp == 1 || (G == 2 && warp == Cfg::MMA_B_WARP)) {
    // ------------------------------------------------------------------ MMA issue
    // One warp per query block.  The whole warp walks an event loop: three lanes
    // test the three barriers that the next products wait for, all at once, a
    // ballot tells every lane what may be issued, and each burst of instructions
    // is predicated on an elected lane (no branch that only one lane takes).
    const int g = warp == 1 ? 0 : 1;
    const int n_mine = g ? n_b : n_a;
    int s_next = 0;              // next tile whose S_g is to be issued
    int o_next = 0;              // next tile whose P_g V is to be issued
    bool ok = true;
    unsigned long long idle_since = 0;
    int idle_rounds = 0;
#ifdef AT_STAMPS
    const bool stamping = blockIdx.x == 0 && blockIdx.y == 0 && lane == 0;
    int n_stamp = 0;
    long long* ev_buf = stamp_buf + 64 + g * 96;
#endif
    const uint32_t tq = tmem_base + Cfg::TMEM_Q + g * (D / 2);
    const uint32_t ts = tmem_base + Cfg::TMEM_S + g * AT_BN;
    const uint32_t to = tmem_base + Cfg::TMEM_O + g * D;
    // The descriptors of stage 0 and of this block's first P buffer, once: a descriptor holds
    // its address in 16-byte units in its low bits, so those of another stage or buffer are
    // a sum (everything lies below 256 KB, the sum stays inside the field).
    static_assert((AT_STAGES & (AT_STAGES - 1)) == 0, "stages are picked with a mask");
    const uint64_t dk0 = make_smem_desc(smem_u32(kv_s));
    const uint64_t dv0 = make_smem_desc_mn(smem_u32(kv_s + DS * Cfg::SUB_BYTES), Cfg::SUB_BYTES);
    const uint64_t dp0 = make_smem_desc(smem_u32(p_s + (g * 2) * Cfg::P_BYTES));
    while (o_next < n_mine) {
      // lane 0: K/V of the tile S_g wants; lane 1: Q_g in place (first tile) or S_g
      // free; lane 2: P_g written.  Branch-free: one test instruction.
      bool mine = true;
      {
        uint64_t* bar = &kv_full[s_next & (AT_STAGES - 1)];
        uint32_t par = ((uint32_t)(s_next / AT_STAGES)) & 1;
        bool need = s_next < n_mine;
        if (lane == 1) {
          bar = s_next == 0 ? &q_full[g] : &s_empty[g];
          par = s_next == 0 ? 0u : ((((uint32_t)s_next) & 1) ^ 1);
        }
        if (lane == 2) {
          bar = &p_full[g * 2 + (o_next & 1)];
          par = ((uint32_t)(o_next >> 1)) & 1;
          need = true;
        }
        if (need && lane < 3) mine = mbar_test(bar, par);
      }
      const uint32_t ready = __ballot_sync(0xffffffffu, mine);
      bool issued = false;
      tc_fence_after();
      // O_g += P_g V of the next tile
      if (o_next < s_next && (ready >> 2 & 1)) {
        const int t = o_next;
        const int st = t & (AT_STAGES - 1);
        // four products of 16 keys: 32 bytes of a P row, 2 key groups of V each
        static_assert(AT_BN == 64, "one burst covers a key tile");
        tc_mma_burst4_w<true>(to, dp0 + (uint64_t)((t & 1) * (Cfg::P_BYTES >> 4)),
                              dv0 + (uint64_t)(st * (Cfg::KV_BYTES >> 4)), 2, (2 * 1024) >> 4, Cfg::IDESC_R,
                              t > 0 ? 1u : 0u, &o_done[g]);
        // K_t and V_t go back to the producer when the products so far are done
        tc_commit_w(&kv_empty[g * AT_STAGES + st]);
        if (t == n_mine - 1) tc_commit_w(&o_final[g]);
        o_next = t + 1;
        issued = true;
#ifdef AT_STAMPS
        if (stamping && n_stamp < 96 && t >= 8) ev_buf[n_stamp++] = (clock64() << 20) | (t << 8) | (g << 4) | 2;
#endif
      }
      // S_g of the next tile = Q_g K^T.  Not before the product of tile t-2 has been
      // issued: the softmax threads take a complete S_t to mean that the P buffer of
      // tile t-2 has been read, and that O_g holds all but the last product.
      if (s_next < n_mine && o_next + 1 >= s_next && (ready & 1) && (ready >> 1 & 1)) {
        const int t = s_next;
        const uint64_t dkt = dk0 + (uint64_t)((t & (AT_STAGES - 1)) * (Cfg::KV_BYTES >> 4));
        // per product 16 elements of head_dim: 8 columns of Q, 32 bytes of a K row
        if (DS == 1) {
          tc_mma_ta_burst4_w<true>(ts, tq, dkt, 2, Cfg::IDESC_S, 0u, &s_full[g]);
        } else {
#pragma unroll
          for (int ds = 0; ds < DS; ++ds) {
            const uint64_t dk = dkt + (uint64_t)(ds * (Cfg::SUB_BYTES >> 4));
            if (ds + 1 < DS) tc_mma_ta_burst4_w<false>(ts, tq + ds * 32, dk, 2, Cfg::IDESC_S, ds > 0 ? 1u : 0u, nullptr);
            else tc_mma_ta_burst4_w<true>(ts, tq + ds * 32, dk, 2, Cfg::IDESC_S, 1u, &s_full[g]);
          }
        }
        s_next = t + 1;
        issued = true;
        if (t == 0 && g == 0 && lane == 0) { BST(2) }
#ifdef AT_STAMPS
        if (stamping && n_stamp < 96 && t >= 8) ev_buf[n_stamp++] = (clock64() << 20) | (t << 8) | (g << 4) | 1;
#endif
      }
      if (issued) {
        idle_rounds = 0;
        continue;
      }
      __nanosleep(40);   // leave the issue slots of this scheduler to its softmax warps
      if (++idle_rounds >= 64) {   // nothing to do for a while: look at the clock
        const unsigned long long now = now_ns();
        if (idle_rounds == 64) idle_since = now;
        const bool stop = *abort_flag || now - idle_since > TC_WAIT_LIMIT_NS;
        if (__any_sync(0xffffffffu, stop)) {
          ok = false;
          break;
        }
        idle_rounds = 65;
      }
    }
    if (!ok && lane == 0) {
      if (!*abort_flag) atomicCAS(a.error, 0, GB_ERR_AT_TIMEOUT);
      *abort_flag = 1;
    }
  } else {
    // ------------------------------------------------------------------ softmax and store
    // One thread per query row.  What a warp does per tile is a chain (barrier, TMEM load,
    // maximum, exponentials, store, fence, barrier) whose length is set by how many
    // instructions it issues and by their latencies, not by the special-function unit (taking
    // the exponentials out changes nothing; neither does halving either product or leaving
    // out the loads): so every instruction that is not arithmetic on the 64 values counts.
    // (Two threads a row, for four warps per scheduler instead of two, was no faster: the
    // per-tile instructions that do not shrink with the values are then paid twice.)
    constexpr int NSW = Cfg::NSW;
    const int idx = warp - 2;
    const int g = idx / NSW;                       // query block of this warp
    const int q = warp & 3;                        // the TMEM lanes this warp may touch
    const int r = q * 32 + lane;                   // query row inside the block
    const int pos = pos0 + g * AT_BM + r;
    const int rows_mine = g ? rows_b : rows_a;
    const int hi = r < rows_mine ? pos : -1;       // rows beyond the step see nothing
    const int lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const uint32_t o_addr = lane_addr + Cfg::TMEM_O + g * D;
    const uint32_t s_addr = lane_addr + Cfg::TMEM_S + g * AT_BN;
    const int n_mine = g ? n_b : n_a;
    // a tile wholly at or below the block's first position P (and inside every row's
    // window) needs no mask: the first that does is the one whose last key lies beyond P
    const int j_mask = (a.window > 0 || rows_mine < AT_BM) ? 0 : max(0, (pos0 + g * AT_BM + 1) / AT_BN - tile_lo);
    const uint32_t p_row = smem_u32(p_s + (g * 2) * Cfg::P_BYTES + r * 128), p_swz = (uint32_t)(r & 7) << 4;
    float m_used = -INFINITY, l = 0.f;             // base of the exponent (scaled), row sum
    bool ok = true;
#ifdef AT_STAMPS
    const bool stamping = blockIdx.x == 0 && blockIdx.y == 0 && lane == 0 && q == 1;
#endif

    auto wait_warp = [&](uint64_t* bar, uint32_t parity) -> bool {
      return mbar_wait_warp(bar, parity, nullptr);
    };
    if (n_mine > 0) {
      // this thread's query row into its lane of tensor memory: 32-bit word c of
      // the row (elements 2c and 2c+1) is column c
      const uint4* qrow = reinterpret_cast<const uint4*>(
          q_rows + ((size_t)(tok0 + g * AT_BM + r) * a.nq + h) * D);
      const uint32_t q_addr = lane_addr + Cfg::TMEM_Q + g * (D / 2);
#pragma unroll
      for (int c0 = 0; c0 < D / 2; c0 += 16) {
        uint32_t v[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 w = make_uint4(0u, 0u, 0u, 0u);
          if (r < rows_mine) w = qrow[c0 / 4 + i];   // rows beyond the step are never read
          v[4 * i] = w.x, v[4 * i + 1] = w.y, v[4 * i + 2] = w.z, v[4 * i + 3] = w.w;
        }
        tc_st16(q_addr + c0, v);
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      mbar_arrive_if(&q_full[g], lane == 0);
    }

    for (int j = 0; j < n_mine; ++j) {
      const int b = j & 1;
      float s[AT_BN];
      float mx;
      const int key0 = (tile_lo + j) * AT_BN;
      const bool need_mask = j >= j_mask;
      AT_STAMP(stamp_buf, (g * 4 + (j - 8)) * 8 + 0)
      if (!wait_warp(&s_full[g], ((uint32_t)j) & 1)) { ok = false; break; }
      {
        tc_fence_after();
        AT_STAMP(stamp_buf, (g * 4 + (j - 8)) * 8 + 1)
        {
          uint32_t v[AT_BN];
          tc_ld64(s_addr, v);
          tc_wait_ld();
#pragma unroll
          for (int jj = 0; jj < AT_BN; ++jj) s[jj] = __uint_as_float(v[jj]);
        }
        tc_fence_before();
        __syncwarp();
        mbar_arrive_if(&s_empty[g], lane == 0);   // S is in registers: the next S may be written
        AT_STAMP(stamp_buf, (g * 4 + (j - 8)) * 8 + 2)
        if (need_mask) {
          const int last = hi - key0, first = lo - key0;   // this row's keys of the tile
          if (a.window > 0) {
#pragma unroll
            for (int c = 0; c < AT_BN; ++c)
              if (c < first || c > last) s[c] = -INFINITY;
          } else {
#pragma unroll
            for (int c = 0; c < AT_BN; ++c)
              if (c > last) s[c] = -INFINITY;
          }
        }
        // (the accumulators start from the first values, not from constants that would
        // have to be loaded into registers every tile)
        float mx4[4] = {fmaxf(s[0], s[1]), fmaxf(s[2], s[3]), fmaxf(s[4], s[5]), fmaxf(s[6], s[7])};
#pragma unroll
        for (int c = 8; c < AT_BN; c += 8) {
          mx4[0] = max3(mx4[0], s[c], s[c + 1]);
          mx4[1] = max3(mx4[1], s[c + 2], s[c + 3]);
          mx4[2] = max3(mx4[2], s[c + 4], s[c + 5]);
          mx4[3] = max3(mx4[3], s[c + 6], s[c + 7]);
        }
        mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * a.scale_log2;
      }

      // raise the base only when the maximum outgrew it by 2^8 (or on the first keys)
      float factor = 1.0f;
      const bool raise = mx > m_used + 8.0f;       // also true when m_used is -inf and mx is finite
      if (raise) {
        factor = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - mx);
        m_used = mx;
      }
      // rows of O that already hold products must be rescaled; the load and store of
      // tensor memory are warp-wide, so the warp does it when any lane has to
      const bool rescale = __any_sync(0xffffffffu, raise && j > 0 && factor != 0.f);
      if (rescale) {
        // S_j is complete, so the product of tile j-2, issued before it, is too:
        // o_done is at most one phase behind
        if (!wait_warp(&o_done[g], ((uint32_t)(j - 1)) & 1)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 16) {
          uint32_t v[16];
          tc_ld16(o_addr + c0, v);
          tc_wait_ld();
#pragma unroll
          for (int jj = 0; jj < 16; ++jj) v[jj] = __float_as_uint(__uint_as_float(v[jj]) * factor);
          tc_st16(o_addr + c0, v);
        }
        tc_wait_st();
        tc_fence_before();
      }
      l *= factor;
      AT_STAMP(stamp_buf, (g * 4 + (j - 8)) * 8 + 3)

      const float mbase = (m_used == -INFINITY) ? 0.f : m_used;
      uint64_t sum4[4];                                  // four pairs of partial sums
      uint32_t pk[AT_BN / 2];
      const uint64_t scale2 = pack_f32x2(a.scale_log2, a.scale_log2), base2 = pack_f32x2(-mbase, -mbase);
#pragma unroll
      for (int c = 0; c < AT_BN; c += 2) {
        float x0, x1;
        unpack_f32x2(fma_f32x2(pack_f32x2(s[c], s[c + 1]), scale2, base2), x0, x1);
        const float e0 = fast_exp2(x0), e1 = fast_exp2(x1);
        if (c < 8) sum4[c >> 1] = pack_f32x2(e0, e1);
        else sum4[(c >> 1) & 3] = add_f32x2(sum4[(c >> 1) & 3], pack_f32x2(e0, e1));
        pk[c / 2] = pack2(e0, e1);
      }
      {
        float lo, hi;
        unpack_f32x2(add_f32x2(add_f32x2(sum4[0], sum4[1]), add_f32x2(sum4[2], sum4[3])), lo, hi);
        l += lo + hi;
      }
      AT_STAMP(stamp_buf, (g * 4 + (j - 8)) * 8 + 4)

      // P into shared memory, K-major [128 rows][64 keys] under the 128-byte swizzle.
      // The buffer is free: S_j was issued after the product of tile j-2, which read
      // this buffer last, and the tensor core completes in order.
      {
        const uint32_t prow = p_row + b * Cfg::P_BYTES;
#pragma unroll
        for (int ch = 0; ch < AT_BN / 8; ++ch)
          sts128(prow + ((uint32_t)(ch << 4) ^ p_swz), pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // visible to the tensor core
      AT_STAMP(stamp_buf, (g * 4 + (j - 8)) * 8 + 6)
      __syncwarp();
      mbar_arrive_if(&p_full[g * 2 + b], lane == 0);
      AT_STAMP(stamp_buf, (g * 4 + (j - 8)) * 8 + 7)
    }

    // (o_done cannot serve here: P is double-buffered, so o_done may be two phases
    // behind and a parity wait would pass on the wrong one)
    if (g == 0 && warp == 2 && lane == 0) { BST(3) }
    if (ok && n_mine > 0) ok = wait_warp(&o_final[g], 0);
    if (!ok) {
      if (lane == 0) {
        atomicCAS(a.error, 0, GB_ERR_AT_TIMEOUT);
        *abort_flag = 1;
      }
    } else if (n_mine > 0) {
      tc_fence_after();
      const float inv = 1.0f / l;
      bf16* orow = a.out + ((size_t)(tok0 + g * AT_BM + r) * a.nq + h) * D;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t v[32];
        tc_ld32(o_addr + c0, v);          // warp-wide: every lane loads, valid rows store
        tc_wait_ld();
        if (r < rows_mine) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 w;
            w.x = pack2(__uint_as_float(v[c]) * inv, __uint_as_float(v[c + 1]) * inv);
            w.y = pack2(__uint_as_float(v[c + 2]) * inv, __uint_as_float(v[c + 3]) * inv);
            w.z = pack2(__uint_as_float(v[c + 4]) * inv, __uint_as_float(v[c + 5]) * inv);
            w.w = pack2(__uint_as_float(v[c + 6]) * inv, __uint_as_float(v[c + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c0 + c) = w;
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  if (warp == 2 && lane == 0) { BST(4) }
  tc_fence_before();
  __syncthreads();
#ifdef AT_BLOCK_STAMPS
  if (threadIdx.x == 0) { BST(5) bst[6] = (unsigned long long)n_tiles; }
#endif
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)Cfg::TMEM_COLS)
                 : "memory");
  }
}

template <int DS, int G>
static int launch(const CUtensorMap& mk, const CUtensorMap& mv, const bf16* q, const AttnTcArgs& a,
                  cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<DS, G>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)AtConfig<DS, G>::SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return gb_launch(attn_prefill_tc_kernel<DS, G>, dim3(a.nq, a.n_qblocks), dim3(AtConfig<DS, G>::THREADS),
                   AtConfig<DS, G>::SMEM, s, mk, mv, q, a);
}

// q [n_tokens, nq, D]; k_pages and v_pages [n_pages, nkv, 64, D]; bf16.
// head_dim 64 or 128 and pages of 64 tokens; anything else is refused
// (GB_ERR_UNSUPPORTED) and the caller uses another kernel.
// rows_per_block 128 or 256: a->n_qblocks counts blocks of that many query rows.
GB_EXPORT int gb_attn_prefill_tc(const void* q, const void* k_pages, const void* v_pages,
                                 const AttnTcArgs* a, int n_tokens, long long n_pages, int D, int page,
                                 int rows_per_block, cudaStream_t s) {
  if (!q || !k_pages || !v_pages || !a->out || !a->error || a->n_seqs <= 0 || a->nq <= 0 ||
      a->nkv <= 0 || a->nq % a->nkv || a->max_pages <= 0 || a->n_qblocks < 0 || n_tokens <= 0 ||
      n_pages <= 0)
    return GB_ERR_BAD_ARG;
  if (page != AT_BN || (D != 64 && D != 128) || a->n_qblocks > 65535) return GB_ERR_UNSUPPORTED;
  if (rows_per_block != AT_BM && rows_per_block != 2 * AT_BM) return GB_ERR_BAD_ARG;
  if (n_pages * a->nkv * AT_BN > 0x7fffffffll) return GB_ERR_UNSUPPORTED;
  if (((uintptr_t)q & 15) != 0) return GB_ERR_BAD_ARG;   // query rows are read 16 bytes at a time
  if (a->n_qblocks == 0) return 0;
  CUtensorMap mk, mv;
  const uint64_t kv_rows = (uint64_t)n_pages * a->nkv * AT_BN;
  int e = tc_make_map_2d(&mk, k_pages, kv_rows, (uint64_t)D, (uint64_t)D * 2, AT_BN, 64);
  if (e) return e;
  e = tc_make_map_2d(&mv, v_pages, kv_rows, (uint64_t)D, (uint64_t)D * 2, AT_BN, 64);
  if (e) return e;
  if (rows_per_block == AT_BM)
    return D == 64 ? launch<1, 1>(mk, mv, (const bf16*)q, *a, s) : launch<2, 1>(mk, mv, (const bf16*)q, *a, s);
  return D == 64 ? launch<1, 2>(mk, mv, (const bf16*)q, *a, s) : launch<2, 2>(mk, mv, (const bf16*)q, *a, s);
}
