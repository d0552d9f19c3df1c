// Attention of single decoded tokens over the paged cache, bf16, split over the
// keys ("split-K") so that a handful of sequences still fills the GPU.
//
// Block (split s, kv head, sequence): the G query heads that share the kv head
// form one 16-row tile (rows >= G are zero); the block's two warps take the
// split's key tiles of 32 keys in turn, each warp streaming its own tiles
// through its own double-buffered shared memory with asynchronous copies, so no
// block-wide barrier sits in the key loop.  The warps' (max, sum, accumulator)
// are merged in shared memory.  With one split the block writes the output;
// otherwise it writes a 32-bit partial (accumulator relative to its max, max,
// sum) to scratch and a second, wide kernel combines the splits in split order:
//   out = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M),  M = max_s m_s.
// The key range of a sequence comes from kv_len on the device, so one captured
// launch serves every step.  (The reference's pair is fmha_decode_gqa_split +
// splitk_reduce_merge, src/kernels.rs:2586-2749, 2771-2868, which stores f16
// partials; these stay 32-bit.)
#include "attn_mma.cuh"

#ifndef DC_BN
#define DC_BN 32       // keys per tile
#endif
#ifndef DC_STAGES
#define DC_STAGES 2    // tiles of a warp in shared memory (one less in flight)
#endif
#define DC_WARPS 2
#define DC_THREADS (DC_WARPS * 32)

struct DecodeArgs {
  const bf16* q;           // [n_seqs, nq, D]
  const bf16* k_pages;     // [n_pages, nkv, page, D]
  const bf16* v_pages;
  const int* block_table;  // [slots, max_pages]
  const int* slots;        // [n_seqs]
  const int* kv_len;       // [n_seqs] keys 0..kv_len-1 exist; the query sits at kv_len-1
  bf16* out;               // [n_seqs, nq, D]
  float* part_o;           // [n_seqs, nq, n_splits, D]   (n_splits > 1)
  float* part_ml;          // [n_seqs, nq, n_splits, 2]
  int n_seqs, nq, nkv, max_pages, page, window, n_splits;
  float scale_log2;
};

template <int DT>
__global__ void __launch_bounds__(DC_THREADS) attn_decode_kernel(const DecodeArgs a) {
  constexpr int D = 16 * DT, LD = D + 8, CHUNKS = D / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);       // [16][LD]
  bf16* kv_s = q_s + 16 * LD;                          // per warp: [stages][K, V][DC_BN][LD]
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
  const int tile_lo = key_lo / DC_BN;
  const int n_tiles = kv_len > 0 ? pos / DC_BN - tile_lo + 1 : 0;
  const int per_split = (n_tiles + a.n_splits - 1) / a.n_splits;
  const int t_begin = tile_lo + split * per_split;
  const int t_end = min(tile_lo + n_tiles, t_begin + per_split);
  const bool empty = t_begin >= t_end;   // a padding row, or more splits than tiles
  // The producer kernel of this step wrote the queries and the key and value of
  // position kv_len - 1; everything else this block reads (slots, lengths, block
  // table, older keys) was there before the step.  So the tiles without the
  // newest key are requested before waiting for the producer, and its last
  // microseconds overlap the start of the key stream.
  const int fresh_tile = pos / DC_BN;

  if (empty) {
    pdl_wait();
    if (single) {
      for (int i = tid; i < G * D; i += DC_THREADS)
        a.out[((size_t)seq * a.nq + h0) * D + i] = __float2bfloat16(0.f);
      return;
    }
    for (int i = tid; i < G; i += DC_THREADS) {
      float* ml = a.part_ml + (((size_t)seq * a.nq + h0 + i) * a.n_splits + split) * 2;
      ml[0] = -INFINITY;
      ml[1] = 0.f;
    }
  } else {
    const int* table = a.block_table + (size_t)slot * a.max_pages;
    bf16* my = kv_s + (size_t)warp * DC_STAGES * 2 * DC_BN * LD;
    const int tiles_per_page = a.page / DC_BN;
    // (a shift where it is a power of two, as with this library's pages of 64: the
    // division sat in front of every tile's first copy)
    const int tpp_shift = (tiles_per_page & (tiles_per_page - 1)) == 0 ? __ffs(tiles_per_page) - 1 : -1;

    // Keys and values of a tile are copied, committed and waited for separately: the key
    // buffer of a stage is refilled as soon as the scores of its tile are computed and the
    // value buffer after the P.V product, so that with two buffers of each a tile and a half
    // are in flight on average, not one.  Every thread commits the groups in the order
    // K(0) V(0) K(1) V(1) ..., empty ones included, which is what the wait counts rely on.
    auto load_half = [&](int tile, int stage, int which) {
      if (tile < t_end) {
        const int pg = tpp_shift >= 0 ? tile >> tpp_shift : tile / tiles_per_page;
        const int in_page = tile - pg * tiles_per_page;
        const int page = table[pg];
        const size_t base = (((size_t)page * a.nkv + kvh) * a.page + in_page * DC_BN) * D;
        bf16* dst = my + (stage * 2 + which) * DC_BN * LD;
        const bf16* src = which ? a.v_pages : a.k_pages;
        const int valid = kv_len - tile * DC_BN;
        for (int i = lane; i < DC_BN * CHUNKS; i += 32) {
          const int r = i / CHUNKS, ch = i % CHUNKS;
          const bool ok = r < valid;
          cp_async16(dst + r * LD + ch * 8, ok ? src + base + r * D + ch * 8 : src, ok);
        }
      }
      cp_async_commit();
    };
    // the first tiles of this warp, then the producer, then the query tile.  A tile that
    // holds the newest key comes last in its warp's list, so issuing what may be issued
    // before the wait keeps the order of the groups.
    const int first = t_begin + warp;
    bool early[DC_STAGES];
#pragma unroll
    for (int s = 0; s < DC_STAGES; ++s) {
      const int tile = first + s * DC_WARPS;
      early[s] = tile >= t_end || tile != fresh_tile;
      if (early[s]) {
        load_half(tile, s, 0);
        load_half(tile, s, 1);
      }
    }
    pdl_wait();
    // the query tile: G rows, the rest zero
    {
      const bf16* qsrc = a.q + ((size_t)seq * a.nq + h0) * D;
      for (int i = tid; i < 16 * CHUNKS; i += DC_THREADS) {
        const int r = i / CHUNKS, ch = i % CHUNKS;
        const bool ok = r < G;
        cp_async16(q_s + r * LD + ch * 8, ok ? qsrc + r * D + ch * 8 : qsrc, ok);
      }
      cp_async_commit();   // a group of its own; everything so far is waited for before the loop
    }
    WarpAttn<DT> w;
    w.init();
    int lo[2] = {key_lo, key_lo}, hi[2] = {pos, pos};
#pragma unroll
    for (int s = 0; s < DC_STAGES; ++s) {   // what had to wait for the producer
      if (!early[s]) {
        load_half(first + s * DC_WARPS, s, 0);
        load_half(first + s * DC_WARPS, s, 1);
      }
    }
    cp_async_wait<0>();   // the query tile and this warp's first tiles have landed for this thread
    __syncthreads();      // ... and for all threads
    w.load_q(q_s);
    int stage = 0;
    // behind the keys of a tile in the order of the groups: its values and both halves of
    // the DC_STAGES - 1 tiles after it; behind its values, once the next keys are issued: the same count
    constexpr int BEHIND = 2 * DC_STAGES - 1;
    for (int tile = first; tile < t_end; tile += DC_WARPS, stage = stage + 1 == DC_STAGES ? 0 : stage + 1) {
      cp_async_wait<BEHIND>();
      __syncwarp();
      const int key0 = tile * DC_BN;
      const bf16* kt = my + (stage * 2 + 0) * DC_BN * LD;
      const bf16* vt = my + (stage * 2 + 1) * DC_BN * LD;
      const int refill = tile + DC_STAGES * DC_WARPS;
      auto between = [&] {
        __syncwarp();   // all lanes have read the keys
        load_half(refill, stage, 0);
        cp_async_wait<BEHIND>();
        __syncwarp();   // the values have landed for every lane
      };
      if (key0 < key_lo || key0 + DC_BN - 1 > pos)
        w.template tile<DC_BN, true>(kt, vt, key0, lo, hi, a.scale_log2, between);
      else
        w.template tile<DC_BN, false>(kt, vt, key0, lo, hi, a.scale_log2, between);
      __syncwarp();  // all lanes are done with the values before their buffer is refilled
      load_half(refill, stage, 1);
    }
    cp_async_wait<0>();
    pdl_launch_dependents();   // the key stream of this block is over
    w.finish_l();
    __syncthreads();  // every warp has left its buffers: reuse them for the merge

    // merge the warps: per warp m[16], l[16], o[16][D] in shared memory
    float* red = reinterpret_cast<float*>(kv_s);
    float* red_m = red;                               // [warps][16]
    float* red_l = red + DC_WARPS * 16;               // [warps][16]
    float* red_o = red + 2 * DC_WARPS * 16;           // [warps][16][D]
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g + r * 8;
      if (t == 0) {
        red_m[warp * 16 + row] = w.m[r];
        red_l[warp * 16 + row] = w.l[r];
      }
#pragma unroll
      for (int i = 0; i < 2 * DT; ++i) {
        red_o[((size_t)warp * 16 + row) * D + i * 8 + t * 2] = w.o[i][2 * r];
        red_o[((size_t)warp * 16 + row) * D + i * 8 + t * 2 + 1] = w.o[i][2 * r + 1];
      }
    }
    __syncthreads();
    for (int i = tid; i < G * D; i += DC_THREADS) {
      const int row = i / D, d = i % D;
      float M = -INFINITY;
#pragma unroll
      for (int wi = 0; wi < DC_WARPS; ++wi) M = fmaxf(M, red_m[wi * 16 + row]);
      float L = 0.f, O = 0.f;
#pragma unroll
      for (int wi = 0; wi < DC_WARPS; ++wi) {
        const float mw = red_m[wi * 16 + row];
        const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
        L += red_l[wi * 16 + row] * f;
        O += red_o[((size_t)wi * 16 + row) * D + d] * f;
      }
      if (single) {
        a.out[((size_t)seq * a.nq + h0 + row) * D + d] = __float2bfloat16(O / L);
      } else {
        const size_t p = ((size_t)seq * a.nq + h0 + row) * a.n_splits + split;
        a.part_o[p * D + d] = O;
      }
    }
    // the rows' maxima and sums: one thread a row, after the loop (a branch for d == 0
    // inside it would be entered by one lane alone in every other pass)
    if (!single && tid < G) {
      float M = -INFINITY, L = 0.f;
#pragma unroll
      for (int wi = 0; wi < DC_WARPS; ++wi) M = fmaxf(M, red_m[wi * 16 + tid]);
#pragma unroll
      for (int wi = 0; wi < DC_WARPS; ++wi) {
        const float mw = red_m[wi * 16 + tid];
        L += red_l[wi * 16 + tid] * ((mw == -INFINITY) ? 0.f : exp2f(mw - M));
      }
      const size_t p = ((size_t)seq * a.nq + h0 + tid) * a.n_splits + split;
      *reinterpret_cast<float2*>(a.part_ml + p * 2) = make_float2(M, L);
    }
  }
}

// out[seq, h, :] from the splits' partials; one block per (sequence, head).
// A separate, wide launch: the combination is a few hundred independent loads
// per output row, which one block per kv head would have to do alone.
__global__ void attn_decode_merge_kernel(const float* part_o, const float* part_ml,
                                         bf16* __restrict__ out, int n_splits, int D) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  // Loads are requested eight splits at a time and then used in split order: a loop that
  // folds one split after the other makes every load wait for the one before it, a round
  // trip to L2 each, and this kernel is nothing but such loads.
  const size_t p0 = (size_t)blockIdx.x * n_splits;
  const float2* ml = reinterpret_cast<const float2*>(part_ml) + p0;   // (max, sum) of every split
  float M = -INFINITY;
  for (int s0 = 0; s0 < n_splits; s0 += 8) {
    float2 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = ml[s0 + u < n_splits ? s0 + u : n_splits - 1];
#pragma unroll
    for (int u = 0; u < 8; ++u) M = fmaxf(M, v[u].x);
  }
  pdl_launch_dependents_if_large();
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float L = 0.f, O = 0.f;
    for (int s0 = 0; s0 < n_splits; s0 += 8) {
      float2 v[8];
      float o[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int sidx = s0 + u < n_splits ? s0 + u : n_splits - 1;
        v[u] = ml[sidx];
        o[u] = part_o[(p0 + sidx) * D + d];
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (s0 + u < n_splits && v[u].x != -INFINITY) {
          const float f = exp2f(v[u].x - M);
          L += v[u].y * f;
          O += o[u] * f;
        }
      }
    }
    out[(size_t)blockIdx.x * D + d] = __float2bfloat16(L > 0.f ? O / L : 0.f);
  }
}

template <int DT>
static int launch(const DecodeArgs& a, cudaStream_t s) {
  constexpr int D = 16 * DT, LD = D + 8;
  const size_t kv_bytes = (size_t)DC_WARPS * DC_STAGES * 2 * DC_BN * LD * sizeof(bf16);
  const size_t red_bytes = (size_t)(2 * DC_WARPS * 16 + DC_WARPS * 16 * D) * sizeof(float);
  const size_t smem = 16 * LD * sizeof(bf16) + (kv_bytes > red_bytes ? kv_bytes : red_bytes);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<DT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  int e = gb_launch(attn_decode_kernel<DT>, dim3(a.n_splits, a.nkv, a.n_seqs), dim3(DC_THREADS),
                    smem, s, a);
  if (e || a.n_splits == 1) return e;
  return gb_launch(attn_decode_merge_kernel, dim3(a.n_seqs * a.nq), dim3(D < 128 ? D : 128), 0, s,
                   (const float*)a.part_o, (const float*)a.part_ml, a.out, a.n_splits, D);
}

// Refuses (GB_ERR_UNSUPPORTED) head sizes that are no multiple of 16 or above
// 128, groups of more than 16 query heads per kv head, and pages that are no
// multiple of 32 tokens; the caller then uses the plain kernel.
GB_EXPORT int gb_attn_decode_bf16(const DecodeArgs* a, int D, cudaStream_t s) {
  if (a->n_seqs < 0 || a->nq <= 0 || a->nkv <= 0 || a->nq % a->nkv || a->max_pages <= 0 ||
      a->n_splits <= 0)
    return GB_ERR_BAD_ARG;
  if (a->n_splits > 1 && (!a->part_o || !a->part_ml)) return GB_ERR_BAD_ARG;
  if (D % 16 || D < 16 || D > 128 || a->nq / a->nkv > 16 || a->page % DC_BN) return GB_ERR_UNSUPPORTED;
  if (a->n_seqs > 65535 || a->nkv > 65535) return GB_ERR_UNSUPPORTED;
  if (a->n_seqs == 0) return 0;
  switch (D / 16) {
    case 1: return launch<1>(*a, s);
    case 2: return launch<2>(*a, s);
    case 3: return launch<3>(*a, s);
    case 4: return launch<4>(*a, s);
    case 5: return launch<5>(*a, s);
    case 6: return launch<6>(*a, s);
    case 7: return launch<7>(*a, s);
    case 8: return launch<8>(*a, s);
  }
  return GB_ERR_UNSUPPORTED;
}
