// bf16 matrix product on the fifth-generation tensor cores:
//   C[rowsA, rowsB] = A[rowsA, K] . B[rowsB, K]^T,  32-bit accumulate,
// with both operands K-major (row-major [rows, K]), which is how activations
// [tokens, in] and weights [out, in] are stored.  The same kernel serves
//   prefill:  A = activations, B = weights, out[token, feature]          and
//   decode:   A = weights, B = the few activation rows, out transposed,
// so that the long dimension always fills the 128 rows of the MMA ("swap A/B").
// The reference calls cuBLAS GemmEx for these products (src/cublas.rs:287-307).
//
// Structure (one persistent block of 192 threads per SM):
//   warp 0    one lane issues TMA loads (cp.async.bulk.tensor.2d, 128-byte
//             swizzle) of a 128 x 64 tile of A and a BN x 64 tile of B per stage
//             into a ring of STAGES shared-memory stages, signalled by mbarriers;
//   warp 1    allocates tensor memory; one lane issues tcgen05.mma
//             (cta_group::1, kind::f16, M = 128, N = BN, K = 16, four per stage)
//             with the accumulator in TMEM, and tcgen05.commit to free the stage;
//   warps 2-5 read the accumulator back with tcgen05.ld (each warp its 32 lanes),
//             convert and store.  Two accumulators alternate, so the epilogue of
//             one tile overlaps the main loop of the next.
// No TMA load uses cluster multicast.
//
// Work split ("stream-K"): tiles x k-blocks form one line of U units; block p
// takes [p U / P, (p + 1) U / P).  A tile covered by one block is written
// directly; a tile shared by several is finished by the block that arrives last
// at the tile's counter, which adds the 32-bit partials (kept in scratch, two
// slots per block) in block order.  No block waits for another block.
//
// One tile per block: when a product has more tiles than the GPU has SMs but all of them
// fit on it at once (two or three blocks an SM), the launch has as many blocks as tiles
// and the rule above gives every block exactly one whole tile; nothing is shared.
//
// Leftover deal (lead_share = S > 0, chosen by the host when there are a few more tiles
// than blocks and the tiles do not all fit at once): block p owns tile p whole, and the tiles beyond the
// P-th are cut S ways over K among blocks 0 .. (tiles - P) S - 1, each of which takes
// its share BEFORE its own tile.  The shares end early and together, so the block that
// adds them does it while its own tile streams, and no block streams two whole tiles.
//
// Every wait on an mbarrier is bounded by a wall-clock limit; when it expires
// the block records a code in args.error, stops issuing work, waits (bounded)
// for its copies in flight, frees its tensor memory and returns.
#include "tc_common.cuh"

// Stages of the ring for tiles of 16, 32 and 64 activation rows.  Six, not as many as
// shared memory holds: with six (109 KB at 16 rows) two blocks fit on an SM, and the blocks
// of the next product start requesting weights while this product's blocks are still in
// their epilogues.  Measured on the whole decode step at batch 8: 8 stages 2.87 ms, 7: 2.86,
// 6: 2.77, 5: 2.83; at batch 64 (one block per SM either way) six is the best too.
#ifndef TC_STAGES_16
#define TC_STAGES_16 6
#endif
#ifndef TC_STAGES_32
#define TC_STAGES_32 6
#endif
#ifndef TC_STAGES_64
#define TC_STAGES_64 6
#endif
#ifndef TC_SHARE_16
#define TC_SHARE_16 6
#endif
#ifndef TC_SHARE_32
#define TC_SHARE_32 4
#endif
#ifndef TC_SHARE_64
#define TC_SHARE_64 4
#endif
// Leftover deal: the most shares a leftover tile is cut into.  The block that adds the
// shares reads them (128 x BN floats each) while its own tile streams; its loads wait
// behind that stream, so wide tiles take few shares.
#ifndef TC_LEAD_SHARE_16
#define TC_LEAD_SHARE_16 10
#endif
#ifndef TC_LEAD_SHARE_32
#define TC_LEAD_SHARE_32 6
#endif
#ifndef TC_LEAD_SHARE_64
#define TC_LEAD_SHARE_64 4
#endif
#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192

#define GB_ERR_TIMEOUT_FULL 101    // MMA warp: a stage never arrived
#define GB_ERR_TIMEOUT_EMPTY 102   // producer: a stage was never released
#define GB_ERR_TIMEOUT_TMEM_FULL 103
#define GB_ERR_TIMEOUT_TMEM_EMPTY 104

struct TcArgs {
  void* out;            // [rowsA, ld] or, transposed, [rowsB, ld]
  float* scratch;       // [2 * blocks][128][BN] partial tiles
  unsigned* counters;   // [tiles], zero before the first launch
  int* error;           // device int, 0 while all is well
  int rowsA, rowsB, K, ld;
  int transpose_out, out_f32;
  int silu;             // transposed output only: rows of A are gate|up interleaved in eights
  int dep_b;            // which operand an earlier kernel writes: 1 = B, 0 = A
  unsigned long long* stamps;   // optional [blocks][8] %globaltimer stamps of the phases, or null
  int split_k;          // > 0: plain split-K, see below
};

// split_k = S > 0 (transposed 32-bit output only): the grid is tiles x S blocks,
// block (tile, s) multiplies the s-th share of K and stores its 32-bit partial at
// out + s * rowsB * ld; nothing is reduced here.  The kernel that consumes the
// product (the residual add of the next norm, the q/k preparation) adds the S
// partials in order.  This takes the whole fixup (partial store, fence, counter,
// reload) off the end of the small projections of a decode step.

#define TC_STAMP(slot)                                                       \
  do {                                                                       \
    if (a.stamps) a.stamps[(size_t)blockIdx.x * 8 + (slot)] = now_ns();      \
  } while (0)

// Stores that are predicated instructions, never a branch.
__device__ __forceinline__ void st_f32_if(float* p, float v, bool on) {
  asm volatile("{ .reg .pred q; setp.ne.b32 q, %2, 0; @q st.global.f32 [%0], %1; }" ::"l"(p), "f"(v),
               "r"((int)on)
               : "memory");
}
__device__ __forceinline__ void st_bf16_if(bf16* p, bf16 v, bool on) {
  asm volatile("{ .reg .pred q; setp.ne.b32 q, %2, 0; @q st.global.b16 [%0], %1; }" ::"l"(p),
               "h"(__bfloat16_as_ushort(v)), "r"((int)on)
               : "memory");
}

__device__ __forceinline__ int tc_block_of_unit(long long u, long long U, int P) {
  return (int)(((u + 1) * P - 1) / U);
}

// The units [rb0, re0) and then [rb1, re1) of the line (tile-major, k-blocks within a tile)
// that block p of P works, for the three ways of dealing: split_k > 0 (block p = tile * S + s
// takes the s-th share of its tile's k-blocks), the leftover deal (lead_share > 0: tile p
// whole, before it a share of one of the tiles beyond the P-th), else equal shares of the
// line.  Host and device use the same function; a host-side test checks that the blocks of
// a launch cover every unit exactly once.  Returns the share's index within its tile in a
// split-K launch, else 0.
__host__ __device__ inline int tc_ranges(int p, int P, int tiles, int kblocks, int split_k, int lead_share,
                                         long long& rb0, long long& re0, long long& rb1, long long& re1) {
  // (the shares of one tile are cut in 32-bit arithmetic: share * kblocks is far below 2^31,
  // and a 64-bit division costs every thread of every block a hundred cycles at its start)
  rb0 = re0 = 0;
  if (split_k > 0) {
    const int tile = p / split_k, sh = p - tile * split_k;
    rb1 = (long long)tile * kblocks + sh * kblocks / split_k;
    re1 = (long long)tile * kblocks + (sh + 1) * kblocks / split_k;
    return sh;
  }
  if (lead_share > 0) {
    rb1 = (long long)p * kblocks;
    re1 = rb1 + kblocks;
    const int n_left = tiles - P;
    if (p < n_left * lead_share) {
      const int j = p / lead_share, sh = p - j * lead_share;
      rb0 = (long long)(P + j) * kblocks + sh * kblocks / lead_share;
      re0 = (long long)(P + j) * kblocks + (sh + 1) * kblocks / lead_share;
    }
    return 0;
  }
  const long long U = (long long)tiles * kblocks;
  rb1 = p * U / P;
  re1 = (p + 1) * U / P;
  return 0;
}

// LEAN: four stages for the tiles of up to 64 columns, so that one more block fits on an SM
// (two of the 32- and 64-column tiles, three of the 16-column ones).  A launch with a few
// more blocks than the GPU otherwise holds at once then runs in one go instead of two
// waves: the qkv product of the widest model at batch 64, 80 tiles cut in two, took 36 us
// as 80 blocks (44 % of the copy peak) and takes 21 as 160.  Where the blocks fit anyway the
// products keep six stages: with four, a gate|up product went from 102 to 117 us.
template <int BN, int LEAN = 0>
struct TcConfig {
  static constexpr int A_BYTES = TC_BM * TC_BK * 2;
  static constexpr int B_BYTES = BN * TC_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;   // both multiples of 1024
  // (wide tiles: as deep a ring as shared memory allows; narrow ones: see TC_STAGES_16)
  static constexpr int STAGES =
      (LEAN && BN <= 64) ? 4
      : BN >= 256 ? 4 : (BN >= 128 ? 6 : (BN >= 64 ? TC_STAGES_64 : (BN >= 32 ? TC_STAGES_32 : TC_STAGES_16)));
  static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
  // Staging for the fused gate|up epilogue of the 32- and 64-column tiles: [BN tokens][64
  // features] bf16 (see the epilogue).
  static constexpr int EPI_BYTES = (BN == 32 || BN == 64) ? BN * 128 : 0;
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 + EPI_BYTES;
  // instruction descriptor: f32 accumulate, bf16 x bf16, both K-major, N = BN, M = 128
  static constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                    ((uint32_t)(TC_BM >> 4) << 24);
};

template <int BN, int LEAN = 0>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const TcArgs a, const int lead_share) {
  using Cfg = TcConfig<BN, LEAN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles_base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(tiles_base + (size_t)STAGES * Cfg::STAGE_BYTES);
  uint64_t* full = bars;                    // [STAGES]
  uint64_t* empty = bars + STAGES;          // [STAGES]
  uint64_t* acc_full = bars + 2 * STAGES;   // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint8_t* epi_s = (uint8_t*)bars + 256;    // [BN][64] bf16, wide tiles with the gate|up epilogue only
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ int last_s;
  volatile int* abort_flag = &abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int P = gridDim.x, p = blockIdx.x;
  if (threadIdx.x == 0) TC_STAMP(0);
  const int tiles_a = (a.rowsA + TC_BM - 1) / TC_BM, tiles_b = (a.rowsB + BN - 1) / BN;
  const int kblocks = (a.K + TC_BK - 1) / TC_BK;
  const long long U = (long long)tiles_a * tiles_b * kblocks;
  // the units of this block: two ranges of the line, worked in this order (the first is
  // empty except in the leftover deal)
  // (scalars, not arrays: an array indexed by the range would live in local memory)
  long long rb0, re0, rb1, re1;
  // (split_index: which share of its tile's k-blocks, in a split-K launch)
  const int split_index = tc_ranges(p, P, tiles_a * tiles_b, kblocks, a.split_k, lead_share, rb0, re0, rb1, re1);

  if (threadIdx.x == 0) {
    tma_prefetch_map(&map_a);
    tma_prefetch_map(&map_b);   // used only after the wait for the producer: have it ready by then
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);   // one arrival per epilogue warp
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
  if (threadIdx.x == 0) TC_STAMP(1);

  // Only the producer lane waits for the kernel before this one (see below): the
  // MMAs need its loads and the epilogue needs the MMAs, so nothing here reads or
  // writes global memory before that wait has returned.
  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      const long long n_units = (re0 - rb0) + (re1 - rb1);
      // The operand that no kernel writes (the weights) is requested for the first
      // ring of stages before this kernel waits for its producer; the other
      // operand (the activations) follows once that kernel has finished.
      const long long n_early = n_units < STAGES ? n_units : STAGES;
      // (tile, k-block) of the unit that is issued next, kept by counting: dividing
      // a 64-bit unit number for every copy cost this lane some 300 cycles a unit
      struct Cursor {
        int ta, tb, kb;
        long long left;   // units left in the first range (0: in the second)
      };
      auto cursor_at = [&](long long u) {
        const int tile = (int)(u / kblocks);
        Cursor c;
        c.kb = (int)(u - (long long)tile * kblocks);
        c.ta = tile % tiles_a;
        c.tb = tile / tiles_a;
        c.left = 0;
        return c;
      };
      auto cursor_first = [&]() {
        if (re0 > rb0) {
          Cursor c = cursor_at(rb0);
          c.left = re0 - rb0;
          return c;
        }
        return cursor_at(rb1);
      };
      auto advance = [&](Cursor& c) {
        if (c.left > 0 && --c.left == 0) {   // the first range is done: on to the second
          c = cursor_at(rb1);
          return;
        }
        if (++c.kb == kblocks) {
          c.kb = 0;
          if (++c.ta == tiles_a) {
            c.ta = 0;
            ++c.tb;
          }
        }
      };
      auto issue = [&](const Cursor& c, int s, bool want_a, bool want_b) {
        uint8_t* sa = tiles_base + (size_t)s * Cfg::STAGE_BYTES;
        if (want_a) tma_load_2d(sa, &map_a, c.kb * TC_BK, c.ta * TC_BM, &full[s]);
        if (want_b) tma_load_2d(sa + Cfg::A_BYTES, &map_b, c.kb * TC_BK, c.tb * BN, &full[s]);
      };
      Cursor cur = cursor_first();
      for (int i = 0; i < (int)n_early; ++i) {   // first round: every stage is free
        mbar_expect_tx(&full[i], Cfg::STAGE_BYTES);
        issue(cur, i, a.dep_b != 0, a.dep_b == 0);
        advance(cur);
      }
      pdl_wait();
      TC_STAMP(2);
      cur = cursor_first();
      for (int i = 0; i < (int)n_early; ++i) {
        issue(cur, i, a.dep_b == 0, a.dep_b != 0);
        advance(cur);
      }
      bool ok = true;
      long long it = n_early;
      int s = (int)(n_early % STAGES);
      uint32_t round = (uint32_t)(n_early / STAGES);
      for (; it < n_units; ++it) {
        if (!mbar_wait(&empty[s], (round & 1) ^ 1, abort_flag)) {
          if (!*abort_flag) atomicCAS(a.error, 0, GB_ERR_TIMEOUT_EMPTY);
          *abort_flag = 1;
          ok = false;
          break;
        }
        mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
        issue(cur, s, true, true);
        advance(cur);
        if (++s == STAGES) {
          s = 0;
          ++round;
        }
      }
      pdl_launch_dependents();
      TC_STAMP(3);
      // Every load issued above completes on a `full` barrier that the MMA warp
      // waits for (or, after an abort, that is waited for below).
      if (!ok) {   // after an abort: let the copies in flight land before the block exits
        for (long long j = max(0ll, it - STAGES); j < it; ++j)
          mbar_wait(&full[j % STAGES], (uint32_t)(j / STAGES) & 1, nullptr, 100000000ull);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue
    if (lane == 0) {
      int s = 0;              // stage and round by counting: every instruction of this
      uint32_t round = 0;     // lane is on the path of the products
      bool first = true;
      int seg = 0;
      bool ok = true;
      // both ranges in turn; the body keeps its indentation, it is one loop over segments
      for (int rg = 0; rg < 2; ++rg)
      for (long long u = rg ? rb1 : rb0, u_end = rg ? re1 : re0; u < u_end && ok; ++seg) {
        const int tile = (int)(u / kblocks);
        const int kb_lo = (int)(u - (long long)tile * kblocks);
        const int kb_hi = (int)min((long long)kblocks, kb_lo + (u_end - u));
        u += kb_hi - kb_lo;
        const int ab = seg & 1;
        if (!mbar_wait(&acc_empty[ab], (((uint32_t)seg >> 1) & 1) ^ 1, abort_flag)) {
          if (!*abort_flag) atomicCAS(a.error, 0, GB_ERR_TIMEOUT_TMEM_EMPTY);
          *abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(ab * BN);
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&full[s], round & 1, abort_flag)) {
            if (!*abort_flag) atomicCAS(a.error, 0, GB_ERR_TIMEOUT_FULL);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          if (first) {
            TC_STAMP(4);
            first = false;
          }
          const uint32_t sa = smem_u32(tiles_base + (size_t)s * Cfg::STAGE_BYTES);
          const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + Cfg::A_BYTES);
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k)   // 16 elements = 32 bytes = 2 descriptor units
            tc_mma(tmem_d, da + 2 * k, db + 2 * k, Cfg::IDESC, (kb > kb_lo || k > 0) ? 1u : 0u);
          tc_commit(&empty[s]);   // the stage is free once these MMAs have read it
          if (++s == STAGES) {
            s = 0;
            ++round;
          }
        }
        if (ok) tc_commit(&acc_full[ab]);
      }
      TC_STAMP(5);
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;               // the TMEM lanes this warp may read
    const int r = q * 32 + lane;          // row of the tile
    const int et = threadIdx.x - 64;      // 0..127 among the epilogue threads
    int seg = 0;
    bool ok = true;
    // (both ranges in turn, as in the MMA lane)
    for (int rg = 0; rg < 2; ++rg)
    for (long long u = rg ? rb1 : rb0, u_end = rg ? re1 : re0; u < u_end && ok; ++seg) {
      const int tile = (int)(u / kblocks);
      const int kb_lo = (int)(u - (long long)tile * kblocks);
      const int kb_hi = (int)min((long long)kblocks, kb_lo + (u_end - u));
      u += kb_hi - kb_lo;
      const int ta = tile % tiles_a, tb = tile / tiles_a;
      const int ab = seg & 1;
      // lane 0 polls for the warp, so that all lanes take the same way; the four
      // epilogue warps wait on the same phase with the same limit and no abort
      // flag, so they agree as well (they meet at a named barrier below)
      int got = 0;
      if (lane == 0) got = mbar_wait(&acc_full[ab], ((uint32_t)seg >> 1) & 1, nullptr) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) {
        if (lane == 0) {
          atomicCAS(a.error, 0, GB_ERR_TIMEOUT_TMEM_FULL);
          *abort_flag = 1;
        }
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(ab * BN);
      const bool whole = a.split_k > 0 || (kb_lo == 0 && kb_hi == kblocks);
      const int row_a = ta * TC_BM + r;
      bool write_out = whole;
      int p_first = 0, p_last = 0;
      if (!whole) {
        // leave the partial [128][BN] in this block's slot, then see who is last
        // slot 0 for the tile this block's own range begins in, slot 1 for its other shared
        // tile (a range ends in at most one more) and for a share of the leftover deal
        const bool my_first_tile = rg == 1 && (int)(rb1 / kblocks) == tile;
        float* mine = a.scratch + ((size_t)2 * p + (my_first_tile ? 0 : 1)) * (size_t)(BN * TC_BM);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          uint32_t v[16];
          tc_ld16(taddr + c0, v);
          tc_wait_ld();
          float4* dst = reinterpret_cast<float4*>(mine + (size_t)r * BN + c0);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            dst[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                 __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[ab]);   // the accumulator may be reused
        const long long t0 = (long long)tile * kblocks;
        if (lead_share > 0) {
          p_first = (tile - P) * lead_share;
          p_last = p_first + lead_share - 1;
        } else {
          p_first = tc_block_of_unit(t0, U, P);
          p_last = tc_block_of_unit(t0 + kblocks - 1, U, P);
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (et == 0) {
          const unsigned old = atomicAdd(&a.counters[tile], 1u);
          last_s = (old == (unsigned)(p_last - p_first));
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        write_out = last_s != 0;
        if (write_out) __threadfence();
      }
      // The gate|up epilogue of a wide tile goes through shared memory: a thread holds one
      // feature of every token, so straight to memory it stores two bytes at a time, 64
      // instructions a thread and 32 bytes a warp each; the tile's [tokens][64 features] is
      // put together in shared memory instead and written as whole 128-byte rows.  (At the
      // 4B sizes and batch 64 the epilogue of the one tile a block has is not hidden behind
      // anything: 3.6 of the product's 22 us.)
      const bool staged = Cfg::EPI_BYTES > 0 && a.transpose_out && a.silu && !a.out_f32 && (a.ld & 7) == 0 &&
                          (((uintptr_t)a.out) & 15) == 0;
      if (write_out) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          float f[16];
          if (whole) {
            uint32_t v[16];
            tc_ld16(taddr + c0, v);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) f[j] = __uint_as_float(v[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) f[j] = 0.f;
            // four contributors' rows are requested at once, then added in block
            // order, so the sum is a fixed one
            for (int qb = p_first; qb <= p_last; qb += 4) {
              float4 t[4][4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int qq = qb + i <= p_last ? qb + i : p_last;
                const bool q_first = lead_share == 0 && (int)(((long long)qq * U / P) / kblocks) == tile;
                const float4* src = reinterpret_cast<const float4*>(
                    a.scratch + ((size_t)2 * qq + (q_first ? 0 : 1)) * (size_t)(BN * TC_BM) +
                    (size_t)r * BN + c0);
#pragma unroll
                for (int k = 0; k < 4; ++k) t[i][k] = __ldcg(src + k);
              }
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                if (qb + i <= p_last) {
#pragma unroll
                  for (int k = 0; k < 4; ++k) {
                    f[4 * k] += t[i][k].x;
                    f[4 * k + 1] += t[i][k].y;
                    f[4 * k + 2] += t[i][k].z;
                    f[4 * k + 3] += t[i][k].w;
                  }
                }
              }
            }
          }
          // store 16 columns of row r
          if (a.transpose_out && a.silu) {
            // rows 16t..16t+7 of A are gates and 16t+8..16t+15 the matching ups: the up
            // of this lane's gate sits 8 lanes further; out[col_b][feature] = silu(g) * u
            // (the reference's silu_mul_2d_f16, src/kernels.rs:271-296, as an epilogue)
            // (addresses advance by one row of the output per column: a running pointer per
            // thread; computing cb * ld afresh for every column went through the uniform
            // datapath and cost about 100 cycles a column)
            const int cb0 = tb * BN + c0;
            const int valid = a.rowsB - cb0;
            const bool mine = (lane & 15) < 8 && row_a < a.rowsA;
            const size_t o0 = (size_t)cb0 * a.ld + (size_t)(row_a >> 4) * 8 + (row_a & 7);
            float* pf = (float*)a.out + o0;
            bf16* pb = (bf16*)a.out + o0;
            const size_t ld = (size_t)a.ld;
            // No branch that only some lanes take: lanes 8-15 and 24-31 compute a value
            // nobody stores, and the store is one predicated instruction.  A branch around
            // the sixteen columns' work, taken by half of each warp, made a chunk of sixteen
            // columns take 2.5 us (a plain chunk: 0.5 us).
            if (a.out_f32) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float up = __shfl_down_sync(0xffffffffu, f[j], 8);
                const float val = __fdividef(f[j], 1.0f + __expf(-f[j])) * up;
                st_f32_if(pf, val, mine && j < valid);
                pf += ld;
              }
            } else if (staged) {
              // feature (r >> 4) * 8 + (r & 7) of token c0 + j (rows and tokens beyond the
              // product's are left out when the rows are written)
              const uint32_t sp = smem_u32(epi_s) + (uint32_t)(c0 * 128 + ((r >> 4) * 8 + (r & 7)) * 2);
              const bool gate_lane = (lane & 15) < 8;
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float up = __shfl_down_sync(0xffffffffu, f[j], 8);
                const float val = __fdividef(f[j], 1.0f + __expf(-f[j])) * up;
                asm volatile("{ .reg .pred q; setp.ne.b32 q, %2, 0; @q st.shared.b16 [%0], %1; }" ::"r"(sp + j * 128),
                             "h"(__bfloat16_as_ushort(__float2bfloat16_rn(val))), "r"((int)gate_lane)
                             : "memory");
              }
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float up = __shfl_down_sync(0xffffffffu, f[j], 8);
                // bf16 output: the fast exponential and division are far inside its rounding
                const float val = __fdividef(f[j], 1.0f + __expf(-f[j])) * up;
                st_bf16_if(pb, __float2bfloat16_rn(val), mine && j < valid);
                pb += ld;
              }
            }
          } else if (a.transpose_out) {
            // out[col_b][row_a]: lanes hold consecutive row_a, so each j is a coalesced store
            if (row_a < a.rowsA) {
              const int cb0 = tb * BN + c0;
              const int valid = a.rowsB - cb0;
              const size_t ld = (size_t)a.ld;
              if (a.out_f32) {
                float* pf = (float*)a.out + (size_t)split_index * a.rowsB * ld + (size_t)cb0 * ld + row_a;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  if (j < valid) *pf = f[j];
                  pf += ld;
                }
              } else {
                bf16* pb = (bf16*)a.out + (size_t)cb0 * ld + row_a;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  if (j < valid) *pb = __float2bfloat16_rn(f[j]);
                  pb += ld;
                }
              }
            }
          } else if (row_a < a.rowsA) {
            const int cb0 = tb * BN + c0;
            const size_t o = (size_t)row_a * a.ld + cb0;
            if (a.out_f32) {
              float* dst = (float*)a.out + o;
              if (cb0 + 16 <= a.rowsB && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
                for (int j = 0; j < 16; j += 4)
                  *reinterpret_cast<float4*>(dst + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
              } else {
                for (int j = 0; j < 16; ++j)
                  if (cb0 + j < a.rowsB) dst[j] = f[j];
              }
            } else {
              bf16* dst = (bf16*)a.out + o;
              if (cb0 + 16 <= a.rowsB && ((uintptr_t)dst & 15) == 0) {
                uint4 w0, w1;
                w0.x = pack2(f[0], f[1]);   w0.y = pack2(f[2], f[3]);
                w0.z = pack2(f[4], f[5]);   w0.w = pack2(f[6], f[7]);
                w1.x = pack2(f[8], f[9]);   w1.y = pack2(f[10], f[11]);
                w1.z = pack2(f[12], f[13]); w1.w = pack2(f[14], f[15]);
                reinterpret_cast<uint4*>(dst)[0] = w0;
                reinterpret_cast<uint4*>(dst)[1] = w1;
              } else {
                for (int j = 0; j < 16; ++j)
                  if (cb0 + j < a.rowsB) dst[j] = __float2bfloat16_rn(f[j]);
              }
            }
          }
        }
        if (staged) {
          asm volatile("bar.sync 1, 128;" ::: "memory");   // the tile is complete in shared memory
          const int feats = a.rowsA >> 1;                  // features of the whole product
          for (int i = et; i < BN * 8; i += 128) {
            const int token = i >> 3, col = tb * BN + token, f0 = ta * (TC_BM / 2) + (i & 7) * 8;
            if (col < a.rowsB && f0 < feats)               // (features come in whole groups of eight)
              *reinterpret_cast<uint4*>((bf16*)a.out + (size_t)col * a.ld + f0) =
                  *reinterpret_cast<const uint4*>(epi_s + token * 128 + (i & 7) * 16);
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");   // before the next tile is staged
        }
        if (!whole && et == 0) a.counters[tile] = 0u;   // ready for the next launch
      }
      if (whole) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[ab]);
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  if (threadIdx.x == 64) TC_STAMP(6);
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) TC_STAMP(7);
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)Cfg::TMEM_COLS)
                 : "memory");
  }
}

// ---- host --------------------------------------------------------------------
// A [rows, K] bf16 row-major operand seen as tiles of box_rows x 64 elements.
static int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  return tc_make_map_2d(map, base, (uint64_t)rows, (uint64_t)K, (uint64_t)K * 2, box_rows, TC_BK);
}

static int pick_bn(int rowsB) {
  if (rowsB <= 16) return 16;
  if (rowsB <= 32) return 32;
  if (rowsB <= 64) return 64;
  if (rowsB <= 128) return 128;
  return 256;
}

struct TcPlan {
  int bn, blocks, scratch_floats, counters;
  int lead_share;   // > 0: the leftover deal with that many shares per leftover tile
  int lean;         // 1: the launch with four stages (TcConfig's LEAN)
};

// Blocks of a tile width that one SM holds at once (by shared memory: 227 KB an SM, a
// kilobyte reserved per block), with the usual ring of stages or the lean one.
static int tc_blocks_per_sm(int bn, bool lean) {
  size_t smem = 0;
  switch (bn) {
    case 16: smem = lean ? TcConfig<16, 1>::SMEM : TcConfig<16>::SMEM; break;
    case 32: smem = lean ? TcConfig<32, 1>::SMEM : TcConfig<32>::SMEM; break;
    case 64: smem = lean ? TcConfig<64, 1>::SMEM : TcConfig<64>::SMEM; break;
    case 128: smem = TcConfig<128>::SMEM; break;
    default: smem = TcConfig<256>::SMEM; break;
  }
  return (int)((227 * 1024) / (smem + 1024));
}

// How many ways K is cut when the consumer adds the partials (split_k mode): as
// many blocks as fill the GPU once, at least four k-blocks each, at most 8 ways.
static int tc_split(int rowsA, int rowsB, int K, int sms) {
  const int bn = rowsB <= 16 ? 16 : (rowsB <= 32 ? 32 : (rowsB <= 64 ? 64 : (rowsB <= 128 ? 128 : 256)));
  const long long tiles = (long long)((rowsA + TC_BM - 1) / TC_BM) * ((rowsB + bn - 1) / bn);
  const int kblocks = (K + TC_BK - 1) / TC_BK;
  long long s = sms / tiles;
#ifndef TC_SPLIT_OVER
#define TC_SPLIT_OVER 6
#endif
  // Two blocks of the tiles of up to 64 columns fit on an SM (the 16-column ones with six
  // stages, the wider ones with the four of TcConfig's LEAN, which a launch with more blocks
  // than SMs takes), so a few more blocks than SMs cost nothing, and one more cut fills the
  // GPU where tiles * s falls well short of it (40 tiles: 160 blocks instead of 120 on 148
  // SMs).  Measured for the wider tiles, decode steps at batch 32 / 64 with and without the
  // extra cut (ms): 4B sizes 3.857 / 5.826 against 3.871 / 5.842, 8B sizes 5.04 / 7.08 against
  // 5.11 / 7.12, 32B sizes 15.08 / 19.38 against 15.33 / 19.51.
  if (bn <= 64 && TC_SPLIT_OVER > 0 &&
      tiles * (s + 1) <= sms + sms / TC_SPLIT_OVER)
    s += 1;
  if (s > kblocks / 4) s = kblocks / 4;
  if (s > 8) s = 8;
  return s < 2 ? 0 : (int)s;   // 0: not worth it (the product already has enough tiles)
}

static int tc_plan_for(int rowsA, int rowsB, int K, int sms, TcPlan* pl);
// SMs of the current device (0 after an error, which the next call reports again).
static int tc_sms(int* err) {
  static int sms = 0;
  *err = 0;
  if (!sms) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) {
      sms = 0;
      *err = (int)e;
    }
  }
  return sms;
}
static int tc_plan(int rowsA, int rowsB, int K, TcPlan* pl) {
  int e = 0;
  const int sms = tc_sms(&e);
  if (e) return e;
  return tc_plan_for(rowsA, rowsB, K, sms, pl);
}
// (the plan for a GPU of `sms` SMs: no device is asked, so a host-side test can call it)
static int tc_plan_for(int rowsA, int rowsB, int K, int sms, TcPlan* pl) {
  const int bn = pick_bn(rowsB);
  const long long tiles = (long long)((rowsA + TC_BM - 1) / TC_BM) * ((rowsB + bn - 1) / bn);
  const long long units = tiles * ((K + TC_BK - 1) / TC_BK);
  if (tiles > (1 << 30)) return GB_ERR_UNSUPPORTED;
  long long blocks = units < sms ? units : sms;
  // The block that finishes a shared tile reads every contributor's partial
  // (128 x BN floats each), one after the other.  With many activation rows that
  // tail outweighs what more blocks gain in streaming, so the number of blocks
  // that may share a tile is capped.
  const long long share = bn <= 16 ? TC_SHARE_16 : (bn <= 32 ? TC_SHARE_32 : TC_SHARE_64);
  if (blocks > tiles * share) blocks = tiles * share;
  // With more tiles than SMs but fewer than one and a half each (152 tiles on 148 SMs:
  // the gate|up product of a decode step), the leftover deal: one whole tile per block and
  // the rest cut over K and taken first.  Measured on that product, in a graph, against
  // the even split of the line above: 18.4 against 21.6 us with 8 activation rows (ten
  // shares), 28.8 against 30.0 us with 64 (four shares; there the even split had already
  // lost to 76 blocks of two whole tiles, which an SM's draw of about 47 GB/s holds back).
  // Failing that, for wide tiles, a number of blocks that divides the tiles, so that no
  // tile is shared.
  pl->lead_share = 0;
  pl->lean = 0;
  if (tiles > sms) {
    const int kblocks = (K + TC_BK - 1) / TC_BK;
    long long s = sms / (tiles - sms);   // as many shares as there are blocks to take them,
    if (s > kblocks / 4) s = kblocks / 4;   // at least four k-blocks each,
    const int most = bn <= 16 ? TC_LEAD_SHARE_16 : (bn <= 32 ? TC_LEAD_SHARE_32 : TC_LEAD_SHARE_64);
    if (s > most) s = most;   // and not more than the adding block reads in passing
    const long long per = (tiles + sms - 1) / sms;
    // More tiles than SMs, but all of them fit on the GPU at once (two or three blocks an
    // SM): one whole tile per block and no tile shared.  The blocks stream side by side and
    // the memory system divides its bandwidth among them, not among the SMs, so the SMs
    // that hold one block more do not finish later.  Measured against the leftover deal
    // below (us exposed inside the decode step; rows x K of the weight, batch): 19,456 x
    // 2,560, 152 tiles: 19.3 against 20.4 at batch 8, 23.1 against 27.3 at batch 64; 24,576
    // x 4,096, 192 tiles: 34.3 against 36.9 at batch 8.
    if (tiles <= (long long)sms * tc_blocks_per_sm(bn, false)) {
      blocks = tiles;
    } else if (bn <= 64 && tiles <= (long long)sms * tc_blocks_per_sm(bn, true)) {
      blocks = tiles;
      pl->lean = 1;
    } else if (tiles < 2 * (long long)sms && s >= 2) {
      blocks = sms;
      pl->lead_share = (int)s;
    } else if (bn >= 64 && tiles % per == 0 && tiles / per >= sms / 2) {
      blocks = tiles / per;
    }
#ifndef TC_NO_WHOLE_TILES
    // Too many tiles for one each even with four stages (400 tiles of 32 or 64 columns: the
    // gate|up product of the widest model): a few whole tiles per block, if the tiles divide
    // so and the blocks then fit at once, rather than equal shares of the line, which share
    // nearly every tile between two blocks.
    if (bn >= 32 && bn <= 64 && tiles > (long long)sms * tc_blocks_per_sm(bn, true)) {
      for (long long k = 2; k <= per + 1; ++k) {
        if (tiles % k) continue;
        const long long b = tiles / k;
        if (b <= sms) {
          blocks = b, pl->lean = 0, pl->lead_share = 0;
          break;
        }
        if (b <= (long long)sms * tc_blocks_per_sm(bn, true)) {
          blocks = b, pl->lean = 1, pl->lead_share = 0;
          break;
        }
      }
    }
#endif
  }
  pl->bn = bn;
  pl->blocks = (int)blocks;
  pl->scratch_floats = (int)(2 * blocks * bn * TC_BM);
  pl->counters = (int)tiles;
  return 0;
}

template <int BN, int LEAN = 0>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, const TcArgs& a, int blocks,
                  int lead_share, cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, LEAN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)TcConfig<BN, LEAN>::SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return gb_launch(gemm_tc_kernel<BN, LEAN>, dim3(blocks), dim3(TC_THREADS), TcConfig<BN, LEAN>::SMEM, s, ma, mb,
                   a, lead_share);
}

static int check_shape(int rowsA, int rowsB, int K) {
  if (rowsA <= 0 || rowsB <= 0 || K <= 0) return GB_ERR_BAD_ARG;
  if (K % 8) return GB_ERR_UNSUPPORTED;   // a row pitch must be a multiple of 16 bytes for TMA
  return 0;
}

// plan[0] = BN, plan[1] = blocks, plan[2] = scratch floats, plan[3] = counters,
// plan[4] = the split count a split_k launch of this shape would use (0: none).
GB_EXPORT int gb_gemm_tc_plan(int rowsA, int rowsB, int K, int* plan) {
  int e = check_shape(rowsA, rowsB, K);
  if (e) return e;
  TcPlan pl;
  e = tc_plan(rowsA, rowsB, K, &pl);
  if (e) return e;
  int sms = 0, dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return GB_ERR_UNSUPPORTED;
  plan[0] = pl.bn;
  plan[1] = pl.blocks;
  plan[2] = pl.scratch_floats;
  plan[3] = pl.counters;
  plan[4] = tc_split(rowsA, rowsB, K, sms);
  return 0;
}

// For host-side tests, no device needed.  plan[0..4] as above for a GPU of `sms` SMs, plan[5] =
// shares of the leftover deal (0: none), plan[6] = 1 for the launch with four stages.
GB_EXPORT int gb_gemm_tc_plan_for(int rowsA, int rowsB, int K, int sms, int* plan) {
  int e = check_shape(rowsA, rowsB, K);
  if (e) return e;
  if (sms <= 0) return GB_ERR_BAD_ARG;
  TcPlan pl;
  e = tc_plan_for(rowsA, rowsB, K, sms, &pl);
  if (e) return e;
  plan[0] = pl.bn, plan[1] = pl.blocks, plan[2] = pl.scratch_floats, plan[3] = pl.counters;
  plan[4] = tc_split(rowsA, rowsB, K, sms);
  plan[5] = pl.lead_share;
  plan[6] = pl.lean;
  return 0;
}
// ranges[0..3] = rb0, re0, rb1, re1 of block p of P (see tc_ranges).
GB_EXPORT int gb_gemm_tc_ranges(int p, int P, int tiles, int kblocks, int split_k, int lead_share,
                                long long* ranges) {
  if (p < 0 || P <= 0 || p >= P || tiles <= 0 || kblocks <= 0) return GB_ERR_BAD_ARG;
  tc_ranges(p, P, tiles, kblocks, split_k, lead_share, ranges[0], ranges[1], ranges[2], ranges[3]);
  return 0;
}

// A [rowsA, K] and B [rowsB, K] bf16, 16-byte aligned; out as TcArgs describes.
GB_EXPORT int gb_gemm_tc_bf16(const void* A, const void* B, const TcArgs* args, cudaStream_t s) {
  int e = check_shape(args->rowsA, args->rowsB, args->K);
  if (e) return e;
  if (!A || !B || !args->out || !args->scratch || !args->counters || !args->error) return GB_ERR_BAD_ARG;
  if ((((uintptr_t)A) | ((uintptr_t)B)) & 15) return GB_ERR_BAD_ARG;
  if (args->silu && (!args->transpose_out || (args->rowsA % 16))) return GB_ERR_UNSUPPORTED;
  TcPlan pl;
  e = tc_plan(args->rowsA, args->rowsB, args->K, &pl);
  if (e) return e;
  bool lean = pl.lean != 0;
  if (args->split_k > 0) {
    if (!args->transpose_out || !args->out_f32 || args->silu) return GB_ERR_UNSUPPORTED;
    const int tiles = ((args->rowsA + TC_BM - 1) / TC_BM) * ((args->rowsB + pl.bn - 1) / pl.bn);
    if (args->split_k > (args->K + TC_BK - 1) / TC_BK) return GB_ERR_BAD_ARG;
    int err = 0;
    // Four stages, two blocks an SM, for the 32- and 64-column tiles: where there are more
    // blocks than SMs, so that they run in one go; and where a block's share of K is short
    // (TC_LEAN_SHARE k-blocks of 64 at most), because the product is then a short kernel between
    // short kernels, and with room for a second block on every SM the next product's blocks
    // are resident and fetching weights while this one's finish (with six stages of 24 KB a
    // block has the SM to itself).  Measured, decode steps at batch 64 (ms, six stages / four
    // for every cut product / four by this rule): Qwen3-4B sizes 5.91 / 5.82, 3.78 / 3.70 with
    // 512 keys a sequence, 3.93 / 3.85 at batch 32; 8B sizes 7.04 / 7.05; 32B sizes 19.39 /
    // 19.86, whose shares are 43 to 133 k-blocks long and want the deeper ring.
#ifndef TC_LEAN_SHARE
#define TC_LEAN_SHARE 32
#endif
    const int share = ((args->K + TC_BK - 1) / TC_BK + args->split_k - 1) / args->split_k;
    lean = (pl.bn == 32 || pl.bn == 64) && (tiles * args->split_k > tc_sms(&err) || share <= TC_LEAN_SHARE);
    pl.blocks = tiles * args->split_k;
    pl.lead_share = 0;
  }
  CUtensorMap ma, mb;
  e = make_map(&ma, A, args->rowsA, args->K, TC_BM);
  if (e) return e;
  e = make_map(&mb, B, args->rowsB, args->K, pl.bn);
  if (e) return e;
  switch (pl.bn) {
    case 16:
      return lean ? launch<16, 1>(ma, mb, *args, pl.blocks, pl.lead_share, s)
                  : launch<16>(ma, mb, *args, pl.blocks, pl.lead_share, s);
    case 32:
      return lean ? launch<32, 1>(ma, mb, *args, pl.blocks, pl.lead_share, s)
                  : launch<32>(ma, mb, *args, pl.blocks, pl.lead_share, s);
    case 64:
      return lean ? launch<64, 1>(ma, mb, *args, pl.blocks, pl.lead_share, s)
                  : launch<64>(ma, mb, *args, pl.blocks, pl.lead_share, s);
    case 128: return launch<128>(ma, mb, *args, pl.blocks, pl.lead_share, s);
    case 256: return launch<256>(ma, mb, *args, pl.blocks, pl.lead_share, s);
  }
  return GB_ERR_UNSUPPORTED;
}

// The way a role of the kernels above gives up, run by itself with nothing in
// flight: no copy is issued, no tensor memory is held, no other block exists.
// Thread 0 waits, for at most limit_ns, on a barrier at which nobody arrives;
// when the time is up it records its code in *error and raises the block's
// abort flag.  Warp 1 waits on a second such barrier with the kernels' own long
// limit and the abort flag, which is what ends its wait.  The block then leaves
// like any other.  It exists so that a test can see the whole path (wait, code,
// abort, return, the host's check) without making a product kernel wait.
__global__ void tc_wait_selftest_kernel(int* error, unsigned long long limit_ns, int* left) {
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ int abort_s;
  volatile int* abort_flag = &abort_s;
  if (threadIdx.x == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    if (!mbar_wait(&bars[0], 0, abort_flag, limit_ns)) {
      if (!*abort_flag) atomicCAS(error, 0, GB_ERR_TIMEOUT_FULL);
      *abort_flag = 1;
    }
  } else if (warp == 1) {
    const bool ok = mbar_wait_warp(&bars[1], 0, abort_flag);
    if (!ok && (threadIdx.x & 31) == 0) atomicAdd(left, 1);   // left because of the abort flag
  }
  __syncthreads();
  if (threadIdx.x == 0) atomicAdd(left, 1);
}
// left: device int that the kernel raises by 2 when both roles have left.
GB_EXPORT int gb_tc_wait_selftest(int* error, long long limit_ns, int* left, cudaStream_t s) {
  if (!error || !left || limit_ns <= 0 || limit_ns > 1000000000ll) return GB_ERR_BAD_ARG;
  tc_wait_selftest_kernel<<<1, 64, 0, s>>>(error, (unsigned long long)limit_ns, left);
  return (int)cudaGetLastError();
}
