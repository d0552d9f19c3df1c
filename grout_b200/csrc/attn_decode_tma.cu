// Attention of single decoded tokens over the paged cache for heads of 64 or 128,
// with the key and value tiles brought in by TMA and the splits of a sequence
// combined by the block that finishes last.
//
// A (page, kv head) pair of the cache is one contiguous tile of 64 keys x D, so
// a tile is one TMA box (two for D = 128) that lands in shared memory under the
// 128-byte swizzle with one instruction of one thread; no thread computes
// addresses or issues 16-byte copies, and the tiles in flight are bounded by
// shared memory alone.  Block (split s, kv head, sequence): the G query heads
// that share the kv head form one 16-row tile (rows >= G are zero); a producer
// lane walks the split's tiles through a ring of STAGES stages (a key barrier
// and a value barrier per stage, so that scores are computed while the values
// are still on their way), the block's two consumer warps take 32 keys of every
// tile each, with their own (max, sum, accumulator), and merge them at the end.
//
// With one split the block writes the output.  Otherwise it writes a 32-bit
// partial (accumulator relative to its max, max, sum) to scratch and counts
// itself in at the (sequence, kv head)'s counter; the block that finds all
// others counted combines the splits in split order,
//   out = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M),  M = max_s m_s,
// and sets the counter back to zero.  No block waits for another.  (The
// reference's pair is fmha_decode_gqa_split + splitk_reduce_merge,
// src/kernels.rs:2586-2749, 2771-2868: two launches and f16 partials.)
//
// The key range of a sequence comes from kv_len on the device, so one captured
// launch serves every step.  Rows of a page beyond the sequence's length are
// masked as keys and zeroed as values in shared memory, so they may hold anything.
// Every barrier wait is bounded (tc_common.cuh); a role that gives up records
// GB_ERR_DECODE_WAIT in *error, the block lets its copies in flight land and
// still counts itself in, so that nothing else is held up.
#include "attn_mma.cuh"
#include "tc_common.cuh"

#define DA_BN 64                    // keys per tile: one page
#define DA_WARPS 2                  // consumer warps; warp DA_WARPS holds the producer lane
#define DA_CONSUMERS (DA_WARPS * 32)
#define DA_THREADS (DA_CONSUMERS + 32)
#define GB_ERR_DECODE_WAIT 131

struct DecodeTmaArgs {
  const bf16* q;           // [n_seqs, nq, D]
  const int* block_table;  // [slots, max_pages]
  const int* slots;        // [n_seqs]
  const int* kv_len;       // [n_seqs] keys 0..kv_len-1 exist; the query sits at kv_len-1
  bf16* out;               // [n_seqs, nq, D]
  float* part_o;           // [n_seqs, nq, n_splits, D]   (n_splits > 1)
  float* part_ml;          // [n_seqs, nq, n_splits, 2]
  int* counters;           // [n_seqs * nkv], zero between launches (n_splits > 1)
  int* error;              // device int, 0 while all is well
  int n_seqs, nq, nkv, max_pages, window, n_splits;
  float scale_log2;
  unsigned long long* stamps;   // optional [blocks][12] %globaltimer stamps of a block's phases (tuning), or null
};

#define DA_STAMP(slot)                                                                          \
  do {                                                                                          \
    if (a.stamps)                                                                               \
      a.stamps[(((size_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 12 + (slot)] = now_ns(); \
  } while (0)

__device__ __forceinline__ void consumer_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(DA_CONSUMERS) : "memory");
}

template <int DS, int STAGES>   // D = 64 * DS
__global__ void __launch_bounds__(DA_THREADS)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const DecodeTmaArgs a) {
  constexpr int D = 64 * DS, DT = D / 16, QLD = D + 8, CHUNKS = D / 8;
  constexpr int HALF_BYTES = DS * DA_BN * 64 * 2;          // the keys (or the values) of a tile
  constexpr int STAGE_BYTES = 2 * HALF_BYTES;
  using Tile = Swizzled128Tile<DA_BN>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* stages = base;                                          // [STAGES][K | V]
  bf16* q_s = reinterpret_cast<bf16*>(base + STAGES * STAGE_BYTES);      // [16][QLD]
  uint64_t* full_k = reinterpret_cast<uint64_t*>(q_s + 16 * QLD);        // [STAGES]
  uint64_t* full_v = full_k + STAGES;
  uint64_t* empty = full_v + STAGES;
  __shared__ int abort_s, issued_s, last_s;
  volatile int* abort_flag = &abort_s;
  volatile int* issued = &issued_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int G = a.nq / a.nkv;
  const int h0 = kvh * G;
  // (both loads at once: the length does not wait for the slot)
  const int slot = a.slots[seq], len_seq = a.kv_len[seq];
  const int kv_len = slot < 0 ? 0 : len_seq;
  const bool single = a.n_splits == 1;

  // key tiles of this split
  const int pos = kv_len - 1;
  const int key_lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
  const int tile_lo = key_lo / DA_BN;
  const int n_tiles = kv_len > 0 ? pos / DA_BN - tile_lo + 1 : 0;
  const int per_split = (n_tiles + a.n_splits - 1) / a.n_splits;
  const int t_begin = tile_lo + split * per_split;
  const int t_end = min(tile_lo + n_tiles, t_begin + per_split);
  const int my_tiles = max(0, t_end - t_begin);
  // The producer kernel of this step wrote the queries and the key and value of
  // position kv_len - 1; everything else this block reads (slots, lengths, block
  // table, older keys) was there before the step.  So the tiles without the
  // newest key are requested before waiting for that kernel.
  const int fresh_tile = pos / DA_BN;

  if (tid == 0) DA_STAMP(0);
  if (tid == DA_CONSUMERS) {      // the producer lane: have the descriptors fetched while the block sets up
    tma_prefetch_map(&map_k);
    tma_prefetch_map(&map_v);
  }
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_k[s], 1);
      mbar_init(&full_v[s], 1);
      mbar_init(&empty[s], DA_WARPS);
    }
    abort_s = 0;
    issued_s = 0;
    last_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == DA_WARPS) {
    // ---- producer: one lane walks the split's tiles through the ring ----------
    if (lane == 0 && my_tiles > 0) {
      const int* table = a.block_table + (size_t)slot * a.max_pages;
      bool waited = false;
      for (int it = 0; it < my_tiles; ++it) {
        const int tile = t_begin + it, s = it % STAGES;
        if (it >= STAGES && !mbar_wait(&empty[s], ((it / STAGES) - 1) & 1, abort_flag)) {
          if (!*abort_flag) atomicCAS(a.error, 0, GB_ERR_DECODE_WAIT);
          *abort_flag = 1;
          break;
        }
        if (*abort_flag) break;
        if (tile == fresh_tile && !waited) {
          pdl_wait();
          waited = true;
        }
        const int row0 = (table[tile] * a.nkv + kvh) * DA_BN;     // first row of the (page, kv head) tile
        unsigned char* st = stages + (size_t)s * STAGE_BYTES;
        mbar_expect_tx(&full_k[s], HALF_BYTES);
#pragma unroll
        for (int ds = 0; ds < DS; ++ds)
          tma_load_2d(st + ds * (DA_BN * 128), &map_k, ds * 64, row0, &full_k[s]);
        mbar_expect_tx(&full_v[s], HALF_BYTES);
#pragma unroll
        for (int ds = 0; ds < DS; ++ds)
          tma_load_2d(st + HALF_BYTES + ds * (DA_BN * 128), &map_v, ds * 64, row0, &full_v[s]);
        *issued = it + 1;
        if (it == 0) DA_STAMP(1);
      }
      DA_STAMP(2);
    }
    return;
  }

  // ---- consumers ----------------------------------------------------------------
  pdl_wait();
  if (tid == 0) DA_STAMP(3);
  WarpAttn<DT> w;
  w.init();
  if (my_tiles > 0) {
    // the query tile: G rows, the rest zero
    const bf16* qsrc = a.q + ((size_t)seq * a.nq + h0) * D;
    for (int i = tid; i < 16 * CHUNKS; i += DA_CONSUMERS) {
      const int r = i / CHUNKS, ch = i % CHUNKS;
      const bool ok = r < G;
      cp_async16(q_s + r * QLD + ch * 8, ok ? qsrc + r * D + ch * 8 : qsrc, ok);
    }
    cp_async_commit();
    cp_async_wait<0>();
    consumer_sync();
    if (tid == 0) DA_STAMP(4);
    w.load_q(q_s);
    int lo[2] = {key_lo, key_lo}, hi[2] = {pos, pos};
    bool ok = true;
    for (int it = 0; it < my_tiles && ok; ++it) {
      const int s = it % STAGES;
      const uint32_t parity = (it / STAGES) & 1;
      const int key0 = (t_begin + it) * DA_BN + warp * 32;    // this warp's 32 keys of the tile
      const bf16* kt = reinterpret_cast<const bf16*>(stages + (size_t)s * STAGE_BYTES);
      bf16* vt = reinterpret_cast<bf16*>(stages + (size_t)s * STAGE_BYTES + HALF_BYTES);
      if (!mbar_wait_warp(&full_k[s], parity, abort_flag)) {
        ok = false;
        break;
      }
      if (tid == 0 && it == 0) DA_STAMP(5);
      const int valid = kv_len - (t_begin + it) * DA_BN;       // rows of the page that hold keys
      bool wrote = false;
      auto between = [&] {
        ok = mbar_wait_warp(&full_v[s], parity, abort_flag);
        if (ok && valid < DA_BN) {
          // rows beyond the sequence: their probabilities are zero, and zero times
          // whatever the page holds there must be zero
          for (int i = lane; i < 32 * CHUNKS; i += 32) {
            const int r = warp * 32 + i / CHUNKS, ch = i % CHUNKS;
            if (r >= valid)
              *reinterpret_cast<uint4*>(vt + Tile::off(r, ch * 8)) = make_uint4(0, 0, 0, 0);
          }
          wrote = true;
          __syncwarp();
        }
      };
      if (key0 < key_lo || key0 + 31 > pos)
        w.template tile<32, true, Tile>(kt, vt, key0, lo, hi, a.scale_log2, between, warp * 32);
      else
        w.template tile<32, false, Tile>(kt, vt, key0, lo, hi, a.scale_log2, between, warp * 32);
      if (!ok) break;          // the values never came: what was added from this tile is void
      // generic-proxy stores into a buffer that the next TMA copy will overwrite
      if (wrote) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
    if (!ok) {
      if (lane == 0) {
        if (!*abort_flag) atomicCAS(a.error, 0, GB_ERR_DECODE_WAIT);
        *abort_flag = 1;
      }
      __syncwarp();
    }
  }
  pdl_launch_dependents();   // the key stream of this block is over
  if (tid == 0) DA_STAMP(6);
  consumer_sync();
  if (*abort_flag && warp == 0 && lane == 0) {
    // let the copies that were issued and not consumed land before the block leaves
    // (bounded; a copy that never lands has already been reported)
    const int n = *issued;
    for (int it = max(0, n - STAGES); it < n; ++it) {
      mbar_wait(&full_k[it % STAGES], (it / STAGES) & 1, nullptr);
      mbar_wait(&full_v[it % STAGES], (it / STAGES) & 1, nullptr);
    }
  }
  consumer_sync();  // every warp has left the stages: reuse them for the merge

  if (my_tiles > 0 && !*abort_flag) {
    w.finish_l();
    // merge the warps: per warp m[16], l[16], o[16][D] in shared memory
    float* red = reinterpret_cast<float*>(stages);
    float* red_m = red;                               // [warps][16]
    float* red_l = red + DA_WARPS * 16;               // [warps][16]
    float* red_o = red + 2 * DA_WARPS * 16;           // [warps][16][D + 8]
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g + r * 8;
      if (row < G) {          // the rows beyond the group's heads are padding: nobody reads them
        if (t == 0) {
          red_m[warp * 16 + row] = w.m[r];
          red_l[warp * 16 + row] = w.l[r];
        }
        // rows are D + 8 floats apart so that the eight rows a warp stores at once fall
        // into different banks
#pragma unroll
        for (int i = 0; i < 2 * DT; ++i)
          *reinterpret_cast<float2*>(red_o + ((size_t)warp * 16 + row) * (D + 8) + i * 8 + t * 2) =
              make_float2(w.o[i][2 * r], w.o[i][2 * r + 1]);
      }
    }
    consumer_sync();
    for (int i = tid; i < G * D; i += DA_CONSUMERS) {
      const int row = i / D, d = i % D;
      float M = -INFINITY;
#pragma unroll
      for (int wi = 0; wi < DA_WARPS; ++wi) M = fmaxf(M, red_m[wi * 16 + row]);
      float L = 0.f, O = 0.f;
#pragma unroll
      for (int wi = 0; wi < DA_WARPS; ++wi) {
        const float mw = red_m[wi * 16 + row];
        const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
        L += red_l[wi * 16 + row] * f;
        O += red_o[((size_t)wi * 16 + row) * (D + 8) + d] * f;
      }
      if (single) {
        a.out[((size_t)seq * a.nq + h0 + row) * D + d] = __float2bfloat16(O / L);
      } else {
        const size_t p = ((size_t)seq * a.nq + h0 + row) * a.n_splits + split;
        a.part_o[p * D + d] = O;
      }
    }
    if (!single && tid < G) {
      float M = -INFINITY, L = 0.f;
#pragma unroll
      for (int wi = 0; wi < DA_WARPS; ++wi) M = fmaxf(M, red_m[wi * 16 + tid]);
#pragma unroll
      for (int wi = 0; wi < DA_WARPS; ++wi) {
        const float mw = red_m[wi * 16 + tid];
        L += red_l[wi * 16 + tid] * ((mw == -INFINITY) ? 0.f : exp2f(mw - M));
      }
      const size_t p = ((size_t)seq * a.nq + h0 + tid) * a.n_splits + split;
      *reinterpret_cast<float2*>(a.part_ml + p * 2) = make_float2(M, L);
    }
  } else {
    // a padding row, more splits than tiles, or a block that gave up: nothing to add
    if (single) {
      for (int i = tid; i < G * D; i += DA_CONSUMERS)
        a.out[((size_t)seq * a.nq + h0) * D + i] = __float2bfloat16(0.f);
    } else {
      for (int i = tid; i < G; i += DA_CONSUMERS) {
        const size_t p = ((size_t)seq * a.nq + h0 + i) * a.n_splits + split;
        *reinterpret_cast<float2*>(a.part_ml + p * 2) = make_float2(-INFINITY, 0.f);
      }
    }
  }
  if (single) return;

  // ---- count in; the block that arrives last combines the splits ------------------
  if (tid == 0) DA_STAMP(7);
  __threadfence();
  consumer_sync();
  if (tid == 0) DA_STAMP(8);
  if (tid == 0) {
    int* counter = a.counters + (size_t)seq * a.nkv + kvh;
    const int before = atomicAdd(counter, 1);
    if (before == a.n_splits - 1) {
      *counter = 0;          // for the next launch; nobody else touches it any more
      last_s = 1;
    }
  }
  consumer_sync();
  if (tid == 0) DA_STAMP(9);
  if (!last_s) return;
  __threadfence();
  // Eight neighbouring columns of one head per thread and pass.  The loads of a pass do
  // not depend on one another (eight splits' maxima, sums and accumulators are requested
  // together and used in split order afterwards), so a pass costs about one trip to L2;
  // head after head, split after split it would cost dozens.
  const int S = a.n_splits;
  constexpr int CPR = D / 8;                       // chunks of eight columns per head
  for (int chunk = tid; chunk < G * CPR; chunk += DA_CONSUMERS) {
    const int row = chunk / CPR, d0 = (chunk % CPR) * 8;
    const size_t p0 = ((size_t)seq * a.nq + h0 + row) * S;
    const float2* ml = reinterpret_cast<const float2*>(a.part_ml) + p0;
    float2 v[8];
    float4 oa[8], ob[8];
    auto request = [&](int s0) {
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int sidx = s0 + u < S ? s0 + u : S - 1;
        const float4* o = reinterpret_cast<const float4*>(a.part_o + (p0 + sidx) * D + d0);
        v[u] = __ldcg(ml + sidx);
        oa[u] = __ldcg(o);
        ob[u] = __ldcg(o + 1);
      }
    };
    request(0);
    float M = -INFINITY;
#pragma unroll
    for (int u = 0; u < 8; ++u) M = fmaxf(M, v[u].x);
    for (int s0 = 8; s0 < S; s0 += 8) {            // more than eight splits: the maximum first
      float2 m2[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) m2[u] = __ldcg(ml + (s0 + u < S ? s0 + u : S - 1));
#pragma unroll
      for (int u = 0; u < 8; ++u) M = fmaxf(M, m2[u].x);
    }
    float L = 0.f, O[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s0 = 0; s0 < S; s0 += 8) {
      if (s0) request(s0);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        // a split without keys left (-inf, 0) and its accumulator unwritten
        if (s0 + u < S && v[u].x != -INFINITY) {
          const float f = exp2f(v[u].x - M);
          L += v[u].y * f;
          O[0] += oa[u].x * f, O[1] += oa[u].y * f, O[2] += oa[u].z * f, O[3] += oa[u].w * f;
          O[4] += ob[u].x * f, O[5] += ob[u].y * f, O[6] += ob[u].z * f, O[7] += ob[u].w * f;
        }
      }
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    uint4 packed;
    packed.x = pack_bf16(O[0] * inv, O[1] * inv);
    packed.y = pack_bf16(O[2] * inv, O[3] * inv);
    packed.z = pack_bf16(O[4] * inv, O[5] * inv);
    packed.w = pack_bf16(O[6] * inv, O[7] * inv);
    *reinterpret_cast<uint4*>(a.out + ((size_t)seq * a.nq + h0 + row) * D + d0) = packed;
  }
  if (tid == 0) DA_STAMP(10);
}

template <int DS, int STAGES>
static size_t smem_bytes() {
  constexpr int D = 64 * DS;
  return 1024 + (size_t)STAGES * 2 * DS * DA_BN * 128 + 16 * (D + 8) * sizeof(bf16) +
         3 * STAGES * sizeof(uint64_t);
}

template <int DS, int STAGES>
static int launch(const CUtensorMap& mk, const CUtensorMap& mv, const DecodeTmaArgs& a,
                  cudaStream_t s) {
  const size_t smem = smem_bytes<DS, STAGES>();
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_tma_kernel<DS, STAGES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return gb_launch(attn_decode_tma_kernel<DS, STAGES>, dim3(a.n_splits, a.nkv, a.n_seqs),
                   dim3(DA_THREADS), smem, s, mk, mv, a);
}

// stages: 2, 3 or 4 tiles of a block in shared memory (0: the default, 3).
// Refuses (GB_ERR_UNSUPPORTED) head sizes other than 64 and 128, groups of more
// than 16 query heads per kv head and pages of other than 64 tokens; the caller
// then uses the kernel without TMA.
GB_EXPORT int gb_attn_decode_tma(const void* k_pages, const void* v_pages, long long n_pages,
                                 const DecodeTmaArgs* a, int D, int page, int stages,
                                 cudaStream_t s) {
  if (a->n_seqs < 0 || a->nq <= 0 || a->nkv <= 0 || a->nq % a->nkv || a->max_pages <= 0 ||
      a->n_splits <= 0 || n_pages <= 0 || !k_pages || !v_pages || !a->error)
    return GB_ERR_BAD_ARG;
  if (a->n_splits > 1 && (!a->part_o || !a->part_ml || !a->counters)) return GB_ERR_BAD_ARG;
  if ((D != 64 && D != 128) || a->nq / a->nkv > 16 || page != DA_BN) return GB_ERR_UNSUPPORTED;
  if (a->n_seqs > 65535 || a->nkv > 65535) return GB_ERR_UNSUPPORTED;
  if (a->n_seqs == 0) return 0;
  const uint64_t rows = (uint64_t)n_pages * a->nkv * page;
  if (rows > 0x7fffffffull) return GB_ERR_UNSUPPORTED;       // TMA coordinates are 32-bit
  CUtensorMap mk, mv;
  int e = tc_make_map_2d(&mk, k_pages, rows, (uint64_t)D, (uint64_t)D * 2, DA_BN, 64);
  if (e) return e;
  e = tc_make_map_2d(&mv, v_pages, rows, (uint64_t)D, (uint64_t)D * 2, DA_BN, 64);
  if (e) return e;
  if (stages == 0) stages = 3;
  if (D == 64) {
    switch (stages) {
      case 2: return launch<1, 2>(mk, mv, *a, s);
      case 3: return launch<1, 3>(mk, mv, *a, s);
      case 4: return launch<1, 4>(mk, mv, *a, s);
    }
  } else {
    switch (stages) {
      case 2: return launch<2, 2>(mk, mv, *a, s);
      case 3: return launch<2, 3>(mk, mv, *a, s);
      case 4: return launch<2, 4>(mk, mv, *a, s);
    }
  }
  return GB_ERR_BAD_ARG;
}
