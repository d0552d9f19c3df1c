// Causal attention of a step's prompt tokens over the paged cache, bf16 with
// 32-bit softmax and accumulation.  One block owns 64 consecutive query rows of
// one sequence and one query head (four warps of 16 rows); key tiles are whole
// pages (64 keys), fetched with asynchronous copies two tiles deep while the
// tensor cores work on the one before.  Queries start at the position that the
// sequence had before the step, so a prompt that continues an earlier one works;
// a window limits every row to its last `window` keys.
//
// Blocks are ordered longest first: the last query block of a long prompt visits
// the most key tiles and is launched first (the idea of the reference's
// fmha_prefill_gqa_lpt, src/kernels.rs:1513-1862).  The reference's kernels are
// cuTile tile programs (src/kernels.rs:1146-1295); this one is written against
// the mma.sync / ldmatrix / cp.async instructions directly.
#include "attn_mma.cuh"

#define PF_BM 64
#define PF_BN 64
#define PF_THREADS 128

struct PrefillArgs {
  const bf16* q;           // [n_tokens, nq, D]
  const bf16* k_pages;     // [n_pages, nkv, 64, D]
  const bf16* v_pages;
  const int* block_table;  // [slots, max_pages]
  const int* cu_q;         // [n_seqs + 1]
  const int* slots;        // [n_seqs]
  const int* kv_len;       // [n_seqs] tokens held after this step
  bf16* out;               // [n_tokens, nq, D]
  int n_seqs, nq, nkv, max_pages, window, n_qblocks;
  float scale_log2;        // scale * log2(e)
};

template <int DT>
__global__ void __launch_bounds__(PF_THREADS) attn_prefill_kernel(const PrefillArgs a) {
  constexpr int D = 16 * DT, LD = D + 8;
  constexpr int CHUNKS = D / 8;  // 16-byte chunks per row
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);  // [64][LD]
  bf16* k_s = q_s + PF_BM * LD;                   // [2][64][LD]
  bf16* v_s = k_s + 2 * PF_BN * LD;               // [2][64][LD]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int h = blockIdx.y;
  const int qb = a.n_qblocks - 1 - blockIdx.x;  // heavy blocks first

  // which sequence does this query block belong to?
  int seq = 0, first_block = 0, q_len = 0;
  for (; seq < a.n_seqs; ++seq) {
    q_len = a.cu_q[seq + 1] - a.cu_q[seq];
    const int nb = (q_len + PF_BM - 1) / PF_BM;
    if (qb < first_block + nb) break;
    first_block += nb;
  }
  if (seq >= a.n_seqs) return;
  const int q0 = (qb - first_block) * PF_BM;       // first row of the block in its sequence
  const int rows = min(PF_BM, q_len - q0);
  const int tok0 = a.cu_q[seq] + q0;               // first row in the step
  const int slot = a.slots[seq];
  bf16* out = a.out + ((size_t)tok0 * a.nq + h) * D;
  const size_t tok_stride = (size_t)a.nq * D;
  if (slot < 0) {  // padding sequence: zeros
    for (int i = tid; i < rows * D; i += PF_THREADS)
      out[(size_t)(i / D) * tok_stride + (i % D)] = __float2bfloat16(0.f);
    return;
  }
  const int kv_len = a.kv_len[seq];
  const int pos0 = kv_len - q_len + q0;            // absolute position of the block's first row
  const int kvh = h / (a.nq / a.nkv);
  const int* table = a.block_table + (size_t)slot * a.max_pages;

  // the block's key range
  const int key_hi = pos0 + rows - 1;
  const int key_lo = (a.window > 0 && pos0 - a.window + 1 > 0) ? pos0 - a.window + 1 : 0;
  const int tile_lo = key_lo / PF_BN, tile_hi = key_hi / PF_BN;

  auto load_tile = [&](int tile, int stage) {
    const int page = table[tile];
    const bf16* ksrc = a.k_pages + ((size_t)page * a.nkv + kvh) * PF_BN * D;
    const bf16* vsrc = a.v_pages + ((size_t)page * a.nkv + kvh) * PF_BN * D;
    bf16* kd = k_s + stage * PF_BN * LD;
    bf16* vd = v_s + stage * PF_BN * LD;
    const int valid = kv_len - tile * PF_BN;  // keys of this page that hold data
    for (int i = tid; i < PF_BN * CHUNKS; i += PF_THREADS) {
      const int r = i / CHUNKS, ch = i % CHUNKS;
      const bool ok = r < valid;  // rows beyond the sequence's length are zero-filled
      cp_async16(kd + r * LD + ch * 8, ok ? ksrc + r * D + ch * 8 : ksrc, ok);
      cp_async16(vd + r * LD + ch * 8, ok ? vsrc + r * D + ch * 8 : vsrc, ok);
    }
  };

  // queries of the block, then the first key tile
  {
    const bf16* qsrc = a.q + ((size_t)tok0 * a.nq + h) * D;
    for (int i = tid; i < PF_BM * CHUNKS; i += PF_THREADS) {
      const int r = i / CHUNKS, ch = i % CHUNKS;
      const bool ok = r < rows;
      cp_async16(q_s + r * LD + ch * 8, ok ? qsrc + (size_t)r * tok_stride + ch * 8 : qsrc, ok);
    }
  }
  load_tile(tile_lo, 0);
  cp_async_commit();

  WarpAttn<DT> w;
  w.init();
  // rows of this lane: warp * 16 + g and + 8
  int lo[2], hi[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + g + r * 8;
    const int pos = pos0 + row;
    hi[r] = row < rows ? pos : -1;  // rows beyond the block see nothing
    lo[r] = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
  }
  // the warp can skip tiles that none of its rows sees
  const int warp_hi = pos0 + min(rows - 1, warp * 16 + 15);
  const int warp_lo = (a.window > 0) ? max(0, pos0 + warp * 16 - a.window + 1) : 0;

  for (int tile = tile_lo; tile <= tile_hi; ++tile) {
    const int stage = (tile - tile_lo) & 1;
    if (tile + 1 <= tile_hi) load_tile(tile + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (tile == tile_lo) w.load_q(q_s + warp * 16 * LD);
    const int key0 = tile * PF_BN;
    if (warp * 16 < rows && key0 <= warp_hi && key0 + PF_BN - 1 >= warp_lo) {
      const bf16* kt = k_s + stage * PF_BN * LD;
      const bf16* vt = v_s + stage * PF_BN * LD;
      // tiles strictly below every row's own position and above every window edge need no mask
      const bool need_mask = (key0 + PF_BN - 1 > pos0 + warp * 16) || (a.window > 0) ||
                             (warp * 16 + 15 >= rows);
      if (need_mask) w.template tile<PF_BN, true>(kt, vt, key0, lo, hi, a.scale_log2);
      else w.template tile<PF_BN, false>(kt, vt, key0, lo, hi, a.scale_log2);
    }
    __syncthreads();  // the stage is refilled two iterations later
  }
  cp_async_wait<0>();
  w.finish_l();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + g + r * 8;
    if (row >= rows) continue;
    const float inv = 1.0f / w.l[r];
    bf16* orow = out + (size_t)row * tok_stride;
#pragma unroll
    for (int i = 0; i < 2 * DT; ++i) {
      const uint32_t v = pack_bf16(w.o[i][2 * r] * inv, w.o[i][2 * r + 1] * inv);
      *reinterpret_cast<uint32_t*>(orow + i * 8 + t * 2) = v;
    }
  }
}

template <int DT>
static int launch(const PrefillArgs& a, cudaStream_t s) {
  constexpr int LD = 16 * DT + 8;
  const size_t smem = (size_t)(PF_BM + 4 * PF_BN) * LD * sizeof(bf16);
  static bool configured = false;  // per instantiation
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<DT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  attn_prefill_kernel<DT><<<dim3(a.n_qblocks, a.nq), PF_THREADS, smem, s>>>(a);
  return gb_status();
}

// head_dim must be a multiple of 16 up to 128 and the page 64 tokens; other
// shapes are refused (the caller then uses the plain kernel).
GB_EXPORT int gb_attn_prefill_bf16(const PrefillArgs* a, int D, int page, cudaStream_t s) {
  if (a->n_seqs <= 0 || a->nq <= 0 || a->nkv <= 0 || a->nq % a->nkv || a->max_pages <= 0 ||
      a->n_qblocks < 0)
    return GB_ERR_BAD_ARG;
  if (page != PF_BN || D % 16 || D < 16 || D > 128) return GB_ERR_UNSUPPORTED;
  if (a->nq > 65535) return GB_ERR_UNSUPPORTED;
  if (a->n_qblocks == 0) return 0;
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
