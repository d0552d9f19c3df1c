// Per (token, head) preparation of the fused q|k|v projection output:
// RMSNorm over head_dim with a weight vector shared by all heads (optional),
// then the half-split rotation of the first `rot_dim` elements (optional), then
// q goes to q_out and k, v go into the paged cache at the token's position
// (and/or to a dense kv_out).  The normalised value is not rounded before the
// rotation: one rounding at the store, as in the reference's
// qk_norm_rope_kv_prefill_raw_f16 (src/kernels.rs:3415-3732, maths 3576-3652).
// angle = float(pos) * inv_freq[j] in 32-bit with the accurate sincosf.
#include "common.cuh"

struct QkPrepareArgs {
  const void* qkv;       // [n_tokens, (nq + 2 nkv) * D]
  const void* q_w;       // [D] or null
  const void* k_w;       // [D] or null
  const float* inv_freq; // [rot_dim / 2] or null
  const int* token_seq;  // [n_tokens] index into slots
  const int* token_pos;  // [n_tokens] absolute position
  const int* slots;      // [n_seqs], < 0 for a padding row
  const int* block_table;
  void* q_out;           // [n_tokens, nq, D]
  void* kv_out;          // [n_tokens, 2 nkv, D] or null
  void* k_pages;         // [n_pages, nkv, page, D] or null
  void* v_pages;
  float eps;
  int n_tokens, nq, nkv, D, rot_dim, max_pages, page;
  const float* qkv_parts;   // instead of qkv: n_parts 32-bit partial sums of it, added in order
  int n_parts;              //   (the split-K projection leaves its reduction to this kernel)
  long long part_stride;    //   floats between partials
};

template <typename T, typename WT>
__global__ void qk_prepare_kernel(const QkPrepareArgs a) {
  extern __shared__ float sm[];
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int n_heads = a.nq + 2 * a.nkv;
  const int head = blockIdx.y * (blockDim.x >> 5) + warp;
  if (head >= n_heads) return;  // warps are independent below
  const int D = a.D;
  float* x = sm + warp * D;
  const T* src = (const T*)a.qkv + ((size_t)t * n_heads + head) * D;
  const int kind = head < a.nq ? 0 : (head < a.nq + a.nkv ? 1 : 2);
  if (a.qkv_parts) {
    const float* ps = a.qkv_parts + ((size_t)t * n_heads + head) * D;
    for (int d = lane; d < D; d += 32) {
      float v = 0.f;
      for (int k = 0; k < a.n_parts; ++k) v += ps[(size_t)k * a.part_stride + d];
      x[d] = v;
    }
  } else {
    for (int d = lane; d < D; d += 32) x[d] = to_f32<T>(src[d]);
  }
  __syncwarp();
  pdl_launch_dependents_if_large();
  const WT* w = kind == 0 ? (const WT*)a.q_w : (kind == 1 ? (const WT*)a.k_w : nullptr);
  if (w) {
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) ss += x[d] * x[d];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)D + a.eps);
    for (int d = lane; d < D; d += 32) x[d] = x[d] * inv * to_f32<WT>(w[d]);
    __syncwarp();
  }
  const int pos = a.token_pos[t];
  if (kind != 2 && a.inv_freq) {
    const int half = a.rot_dim / 2;
    for (int j = lane; j < half; j += 32) {
      const float angle = (float)pos * a.inv_freq[j];
      float s, c;
      sincosf(angle, &s, &c);
      const float lo = x[j], hi = x[j + half];
      x[j] = lo * c - hi * s;
      x[j + half] = hi * c + lo * s;
    }
    __syncwarp();
  }
  if (kind == 0) {
    T* dst = (T*)a.q_out + ((size_t)t * a.nq + head) * D;
    for (int d = lane; d < D; d += 32) dst[d] = from_f32<T>(x[d]);
    return;
  }
  const int hh = kind == 1 ? head - a.nq : head - a.nq - a.nkv;
  if (a.kv_out) {
    T* dst = (T*)a.kv_out + ((size_t)t * 2 * a.nkv + (kind == 1 ? hh : a.nkv + hh)) * D;
    for (int d = lane; d < D; d += 32) dst[d] = from_f32<T>(x[d]);
  }
  if (a.k_pages) {
    const int slot = a.slots[a.token_seq[t]];
    if (slot < 0) return;  // padding row: nothing is stored
    const int* table = a.block_table + (size_t)slot * a.max_pages;
    T* base = (T*)(kind == 1 ? a.k_pages : a.v_pages);
    T* dst = base + paged_row(table, pos, hh, a.nkv, a.page, D);
    for (int d = lane; d < D; d += 32) dst[d] = from_f32<T>(x[d]);
  }
}

// The same work for bf16 heads whose size is a multiple of 64 and that are
// rotated whole (or not at all): a lane keeps its 4 * P elements (pairs 2l, 2l+1
// of each 64-element run, in both halves of the head) in registers, so there is
// no staging in shared memory and all traffic is in 4-byte pieces.
template <typename WT, int P>
__global__ void qk_prepare_fast_kernel(const QkPrepareArgs a) {
  pdl_launch_dependents_if_small();
  // Positions, slots, the block table, the frequencies and the norm weights were in memory
  // before the step began; only the product is the kernel before this one's.  So the
  // position's sines, the page of its key and value and the weights are fetched before the
  // wait for that kernel, and after it only the product's values remain on the path.
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int n_heads = a.nq + 2 * a.nkv;
  const int warps = blockDim.x >> 5;
  constexpr int D = 64 * P, HALF = D / 2;
  constexpr int NP = (P + 1) / 2;   // pairs per half per lane: HALF / 64 rounded up
  // a lane takes the pairs at 2 * lane + 64 * p of each half while they lie inside it
  const int pos = a.token_pos[t];
  // the rotation of a position is the same for every head of the token: once per warp
  float sn[NP][2], cs[NP][2];
  if (a.inv_freq) {
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      const int j = 2 * lane + 64 * p;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        sn[p][e] = 0.f, cs[p][e] = 1.f;
        if (j < HALF) sincosf((float)pos * a.inv_freq[j + e], &sn[p][e], &cs[p][e]);
      }
    }
  }
  size_t page_row0 = 0;   // row of (page of pos, kv head 0, pos in page)
  bool paged = false;
  if (a.k_pages) {
    const int slot = a.slots[a.token_seq[t]];
    if (slot >= 0) {
      page_row0 = paged_row(a.block_table + (size_t)slot * a.max_pages, pos, 0, a.nkv, a.page, D);
      paged = true;
    }
  }
  float wq[NP][4], wk[NP][4];   // the norm weights of this lane's elements, for queries and keys
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    const int j = 2 * lane + 64 * p;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = (e < 2 ? j : HALF + j) + (e & 1);
      wq[p][e] = (j < HALF && a.q_w) ? to_f32<WT>(((const WT*)a.q_w)[idx]) : 1.f;
      wk[p][e] = (j < HALF && a.k_w) ? to_f32<WT>(((const WT*)a.k_w)[idx]) : 1.f;
    }
  }
  pdl_wait();
  // heads of this token in turn: few blocks per token when there are many tokens
  for (int head = blockIdx.y * warps + warp; head < n_heads; head += gridDim.y * warps) {
    const bf16* src = (const bf16*)a.qkv + ((size_t)t * n_heads + head) * D;
    const int kind = head < a.nq ? 0 : (head < a.nq + a.nkv ? 1 : 2);
    float lo[NP][2], hi[NP][2];
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      const int j = 2 * lane + 64 * p;
      if (j < HALF && a.qkv_parts) {
        const float* ps = a.qkv_parts + ((size_t)t * n_heads + head) * D;
        float2 l2 = make_float2(0.f, 0.f), h2 = make_float2(0.f, 0.f);
        // four partials are requested at once and then added in order (one at a time, each
        // load would wait for the one before it to have been added)
        for (int k0 = 0; k0 < a.n_parts; k0 += 4) {
          float2 lk[4], hk[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int k = k0 + u < a.n_parts ? k0 + u : a.n_parts - 1;
            lk[u] = *reinterpret_cast<const float2*>(ps + (size_t)k * a.part_stride + j);
            hk[u] = *reinterpret_cast<const float2*>(ps + (size_t)k * a.part_stride + HALF + j);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (k0 + u < a.n_parts) {
              l2.x += lk[u].x; l2.y += lk[u].y; h2.x += hk[u].x; h2.y += hk[u].y;
            }
        }
        lo[p][0] = l2.x; lo[p][1] = l2.y;
        hi[p][0] = h2.x; hi[p][1] = h2.y;
      } else if (j < HALF) {
        const __nv_bfloat162 l2 = *reinterpret_cast<const __nv_bfloat162*>(src + j);
        const __nv_bfloat162 h2 = *reinterpret_cast<const __nv_bfloat162*>(src + HALF + j);
        lo[p][0] = __low2float(l2); lo[p][1] = __high2float(l2);
        hi[p][0] = __low2float(h2); hi[p][1] = __high2float(h2);
      } else {
        lo[p][0] = lo[p][1] = hi[p][0] = hi[p][1] = 0.f;
      }
    }
    const bool normed = kind == 0 ? a.q_w != nullptr : (kind == 1 && a.k_w != nullptr);
    if (normed) {
      float ss = 0.f;
#pragma unroll
      for (int p = 0; p < NP; ++p)
        ss += lo[p][0] * lo[p][0] + lo[p][1] * lo[p][1] + hi[p][0] * hi[p][0] + hi[p][1] * hi[p][1];
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)D + a.eps);
#pragma unroll
      for (int p = 0; p < NP; ++p) {
        // (beyond the head the values are zero and stay zero)
        lo[p][0] = lo[p][0] * inv * (kind == 0 ? wq[p][0] : wk[p][0]);
        lo[p][1] = lo[p][1] * inv * (kind == 0 ? wq[p][1] : wk[p][1]);
        hi[p][0] = hi[p][0] * inv * (kind == 0 ? wq[p][2] : wk[p][2]);
        hi[p][1] = hi[p][1] * inv * (kind == 0 ? wq[p][3] : wk[p][3]);
      }
    }
    if (kind != 2 && a.inv_freq) {
#pragma unroll
      for (int p = 0; p < NP; ++p) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float l = lo[p][e], h = hi[p][e];
          lo[p][e] = l * cs[p][e] - h * sn[p][e];
          hi[p][e] = h * cs[p][e] + l * sn[p][e];
        }
      }
    }
    bf16* dst = nullptr;
    bf16* dst2 = nullptr;
    if (kind == 0) {
      dst = (bf16*)a.q_out + ((size_t)t * a.nq + head) * D;
    } else {
      const int hh = kind == 1 ? head - a.nq : head - a.nq - a.nkv;
      if (a.kv_out)
        dst2 = (bf16*)a.kv_out + ((size_t)t * 2 * a.nkv + (kind == 1 ? hh : a.nkv + hh)) * D;
      if (paged)
        dst = (bf16*)(kind == 1 ? a.k_pages : a.v_pages) + page_row0 + (size_t)hh * a.page * D;
    }
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      const int j = 2 * lane + 64 * p;
      if (j < HALF) {
        const __nv_bfloat162 l2 = __floats2bfloat162_rn(lo[p][0], lo[p][1]);
        const __nv_bfloat162 h2 = __floats2bfloat162_rn(hi[p][0], hi[p][1]);
        if (dst) {
          *reinterpret_cast<__nv_bfloat162*>(dst + j) = l2;
          *reinterpret_cast<__nv_bfloat162*>(dst + HALF + j) = h2;
        }
        if (dst2) {
          *reinterpret_cast<__nv_bfloat162*>(dst2 + j) = l2;
          *reinterpret_cast<__nv_bfloat162*>(dst2 + HALF + j) = h2;
        }
      }
    }
  }
  pdl_launch_dependents_if_large();
}

// The same again for many tokens (a prompt): the kernel above spends some 25
// instructions an element, which bounds it long before memory does.  Here a lane
// takes 8 consecutive elements of each half of a head in one 16-byte piece, so a
// head is D / 16 lanes and a warp prepares 32 / (D / 16) heads at a time; norm
// weights and the token's rotation are fetched once and reused for every head.
template <typename WT, int P>
__global__ void __launch_bounds__(128, 8) qk_prepare_wide_kernel(const QkPrepareArgs a) {
  // (what does not come from the kernel before this one, the product, is fetched
  // before the wait for it, as in the kernel above)
  constexpr int D = 64 * P, HALF = D / 2, LPH = D / 16, HPW = 32 / LPH;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPH, j0 = 8 * (lane % LPH);
  const int t = blockIdx.x;
  const int n_heads = a.nq + 2 * a.nkv;
  const int warps = blockDim.x >> 5;
  const int pos = a.token_pos[t];
  // the token's rotation: each angle is computed by one thread of the block and
  // shared (an accurate sine and cosine cost some forty instructions)
  // (and so are the norm weights: in registers they would cost the blocks per SM that keep
  // enough loads in flight)
  __shared__ __align__(16) float sn_s[HALF], cs_s[HALF], wq_s[D], wk_s[D];
  for (int j = threadIdx.x; j < HALF; j += blockDim.x) {
    float sj = 0.f, cj = 1.f;
    if (a.inv_freq) sincosf((float)pos * a.inv_freq[j], &sj, &cj);
    sn_s[j] = sj, cs_s[j] = cj;
  }
  for (int j = threadIdx.x; j < D; j += blockDim.x) {
    wq_s[j] = a.q_w ? to_f32<WT>(((const WT*)a.q_w)[j]) : 1.f;
    wk_s[j] = a.k_w ? to_f32<WT>(((const WT*)a.k_w)[j]) : 1.f;
  }
  __syncthreads();
  size_t page_row0 = 0;   // row of (page of pos, kv head 0, pos in page)
  bool paged = false;
  if (a.k_pages) {
    const int slot = a.slots[a.token_seq[t]];
    if (slot >= 0) {
      page_row0 = paged_row(a.block_table + (size_t)slot * a.max_pages, pos, 0, a.nkv, a.page, D);
      paged = true;
    }
  }
  pdl_wait();
  const int passes = (n_heads + HPW - 1) / HPW;
  // A warp's passes in groups of WIDE_U: the loads of a group are all requested before the
  // first of them is used.  One pass at a time left 32 bytes a lane in flight and the
  // kernel at half of the memory's rate.
  constexpr int WIDE_U = 3;
  const int stride = gridDim.y * warps;
  for (int pass0 = blockIdx.y * warps + warp; pass0 < passes; pass0 += WIDE_U * stride) {
  uint4 lo4s[WIDE_U], hi4s[WIDE_U];
#pragma unroll
  for (int u = 0; u < WIDE_U; ++u) {
    const int head = (pass0 + u * stride) * HPW + sub;
    const bool live = pass0 + u * stride < passes && head < n_heads;
    const bf16* src = (const bf16*)a.qkv + ((size_t)t * n_heads + (live ? head : 0)) * D;
    lo4s[u] = *reinterpret_cast<const uint4*>(src + j0);
    hi4s[u] = *reinterpret_cast<const uint4*>(src + HALF + j0);
  }
#pragma unroll
  for (int u = 0; u < WIDE_U; ++u) {
    const int pass = pass0 + u * stride;
    if (pass >= passes) break;            // the same for every lane of the warp
    const int head = pass * HPW + sub;
    const bool live = head < n_heads;     // every lane walks the loop: the sums below are warp-wide
    const uint4 lo4 = lo4s[u], hi4 = hi4s[u];
    float lo[8], hi[8];
    {
      const uint32_t lw[4] = {lo4.x, lo4.y, lo4.z, lo4.w}, hw[4] = {hi4.x, hi4.y, hi4.z, hi4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 l2 = *reinterpret_cast<const __nv_bfloat162*>(&lw[i]);
        const __nv_bfloat162 h2 = *reinterpret_cast<const __nv_bfloat162*>(&hw[i]);
        lo[2 * i] = __low2float(l2), lo[2 * i + 1] = __high2float(l2);
        hi[2 * i] = __low2float(h2), hi[2 * i + 1] = __high2float(h2);
      }
    }
    const int kind = head < a.nq ? 0 : (head < a.nq + a.nkv ? 1 : 2);
    const bool normed = (kind == 0 && a.q_w) || (kind == 1 && a.k_w);
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += lo[e] * lo[e] + hi[e] * hi[e];
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (normed) {
      const float inv = 1.0f / sqrtf(ss / (float)D + a.eps);
      const float* wn = kind == 0 ? wq_s : wk_s;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        lo[e] = lo[e] * inv * wn[j0 + e];
        hi[e] = hi[e] * inv * wn[HALF + j0 + e];
      }
    }
    if (kind != 2 && a.inv_freq) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float l = lo[e], h = hi[e], c = cs_s[j0 + e], sj = sn_s[j0 + e];
        lo[e] = l * c - h * sj;
        hi[e] = h * c + l * sj;
      }
    }
    uint4 lo_o, hi_o;
    {
      uint32_t lw[4], hw[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 l2 = __floats2bfloat162_rn(lo[2 * i], lo[2 * i + 1]);
        const __nv_bfloat162 h2 = __floats2bfloat162_rn(hi[2 * i], hi[2 * i + 1]);
        lw[i] = *reinterpret_cast<const uint32_t*>(&l2);
        hw[i] = *reinterpret_cast<const uint32_t*>(&h2);
      }
      lo_o = make_uint4(lw[0], lw[1], lw[2], lw[3]);
      hi_o = make_uint4(hw[0], hw[1], hw[2], hw[3]);
    }
    if (!live) continue;
    bf16* dst = nullptr;
    bf16* dst2 = nullptr;
    if (kind == 0) {
      dst = (bf16*)a.q_out + ((size_t)t * a.nq + head) * D;
    } else {
      const int hh = kind == 1 ? head - a.nq : head - a.nq - a.nkv;
      if (a.kv_out)
        dst2 = (bf16*)a.kv_out + ((size_t)t * 2 * a.nkv + (kind == 1 ? hh : a.nkv + hh)) * D;
      if (paged)
        dst = (bf16*)(kind == 1 ? a.k_pages : a.v_pages) + page_row0 + (size_t)hh * a.page * D;
    }
    if (dst) {
      *reinterpret_cast<uint4*>(dst + j0) = lo_o;
      *reinterpret_cast<uint4*>(dst + HALF + j0) = hi_o;
    }
    if (dst2) {
      *reinterpret_cast<uint4*>(dst2 + j0) = lo_o;
      *reinterpret_cast<uint4*>(dst2 + HALF + j0) = hi_o;
    }
  }
  }
  pdl_launch_dependents();
}

template <typename WT>
static int launch_wide(const QkPrepareArgs& a, cudaStream_t stream) {
  const int warps = 4;
  dim3 grid(a.n_tokens, 1);
  switch (a.D / 64) {
    case 1: return gb_launch(qk_prepare_wide_kernel<WT, 1>, grid, dim3(warps * 32), 0, stream, a);
    case 2: return gb_launch(qk_prepare_wide_kernel<WT, 2>, grid, dim3(warps * 32), 0, stream, a);
    case 4: return gb_launch(qk_prepare_wide_kernel<WT, 4>, grid, dim3(warps * 32), 0, stream, a);
  }
  return GB_ERR_UNSUPPORTED;
}

// 16-byte pieces need 16-byte addresses: all of them are multiples of 8 elements
// from their tensor's start.
static bool wide_ok(const QkPrepareArgs& a) {
  auto al = [](const void* p) { return (((uintptr_t)p) & 15) == 0; };
  return a.n_tokens >= 128 && !a.qkv_parts && al(a.qkv) && al(a.q_out) && al(a.kv_out) && al(a.k_pages) &&
         al(a.v_pages);
}

template <typename WT>
static int launch_fast(const QkPrepareArgs& a, cudaStream_t stream) {
  const int warps = 4;
  const int n_heads = a.nq + 2 * a.nkv;
  // with few tokens one warp per head; with many, a warp walks several heads and
  // computes the token's rotation once
  const int per_warp = a.n_tokens >= 1024 ? 6 : (a.n_tokens >= 128 ? 2 : 1);
  dim3 grid(a.n_tokens, (n_heads + warps * per_warp - 1) / (warps * per_warp));
  switch (a.D / 64) {
    case 1: return gb_launch(qk_prepare_fast_kernel<WT, 1>, grid, dim3(warps * 32), 0, stream, a);
    case 2: return gb_launch(qk_prepare_fast_kernel<WT, 2>, grid, dim3(warps * 32), 0, stream, a);
    case 4: return gb_launch(qk_prepare_fast_kernel<WT, 4>, grid, dim3(warps * 32), 0, stream, a);
  }
  return GB_ERR_UNSUPPORTED;
}

static bool fast_ok(const QkPrepareArgs& a) {
  return (a.D == 64 || a.D == 128 || a.D == 256) && (!a.inv_freq || a.rot_dim == a.D);
}

template <typename T, typename WT>
static int launch(const QkPrepareArgs& a, cudaStream_t stream) {
  const int warps = 4;
  const int n_heads = a.nq + 2 * a.nkv;
  dim3 grid(a.n_tokens, (n_heads + warps - 1) / warps);
  const size_t smem = (size_t)warps * a.D * sizeof(float);
  if (smem > 48 * 1024) return GB_ERR_UNSUPPORTED;
  return gb_launch(qk_prepare_kernel<T, WT>, grid, dim3(warps * 32), smem, stream, a);
}

static int check(const QkPrepareArgs& a) {
  if (a.n_tokens < 0 || a.nq <= 0 || a.nkv < 0 || a.D <= 0 || (!a.qkv && !a.qkv_parts) || !a.q_out)
    return GB_ERR_BAD_ARG;
  if (a.qkv_parts && (a.n_parts <= 0 || (a.part_stride & 1) || (((uintptr_t)a.qkv_parts) & 7)))
    return GB_ERR_BAD_ARG;
  if (a.inv_freq && (a.rot_dim <= 0 || a.rot_dim > a.D || (a.rot_dim & 1))) return GB_ERR_BAD_ARG;
  if (a.k_pages && (!a.v_pages || !a.block_table || !a.slots || !a.token_seq || a.page <= 0 ||
                    a.max_pages <= 0))
    return GB_ERR_BAD_ARG;
  if (!a.token_pos) return GB_ERR_BAD_ARG;
  return 0;
}

GB_EXPORT int gb_qk_prepare_f32(const QkPrepareArgs* a, int w_is_f32, cudaStream_t s) {
  int e = check(*a);
  if (e) return e;
  if (a->n_tokens == 0) return 0;
  if (!w_is_f32) return GB_ERR_UNSUPPORTED;
  return launch<float, float>(*a, s);
}
GB_EXPORT int gb_qk_prepare_bf16(const QkPrepareArgs* a, int w_is_f32, cudaStream_t s) {
  int e = check(*a);
  if (e) return e;
  if (a->n_tokens == 0) return 0;
  if (fast_ok(*a) && wide_ok(*a)) return w_is_f32 ? launch_wide<float>(*a, s) : launch_wide<bf16>(*a, s);
  if (fast_ok(*a)) return w_is_f32 ? launch_fast<float>(*a, s) : launch_fast<bf16>(*a, s);
  return w_is_f32 ? launch<bf16, float>(*a, s) : launch<bf16, bf16>(*a, s);
}

// Copies dense k, v rows [n_tokens, 2 nkv, D] into the paged cache: the second
// half of the work above for position encodings that are applied outside it.
template <typename T>
__global__ void kv_write_kernel(const T* __restrict__ kv, const int* token_seq,
                                const int* token_pos, const int* slots, const int* block_table,
                                T* k_pages, T* v_pages, int nkv, int D, int max_pages, int page) {
  const int t = blockIdx.x, hh = blockIdx.y;  // hh in [0, 2 nkv)
  const int slot = slots[token_seq[t]];
  if (slot < 0) return;
  const int* table = block_table + (size_t)slot * max_pages;
  const bool is_k = hh < nkv;
  T* dst = (is_k ? k_pages : v_pages) +
           paged_row(table, token_pos[t], is_k ? hh : hh - nkv, nkv, page, D);
  const T* src = kv + ((size_t)t * 2 * nkv + hh) * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) dst[d] = src[d];
}

template <typename T>
static int kv_write(const void* kv, const int* token_seq, const int* token_pos, const int* slots,
                    const int* block_table, void* k_pages, void* v_pages, int n_tokens, int nkv,
                    int D, int max_pages, int page, cudaStream_t s) {
  if (n_tokens < 0 || nkv <= 0 || D <= 0 || page <= 0 || max_pages <= 0) return GB_ERR_BAD_ARG;
  if (n_tokens == 0) return 0;
  kv_write_kernel<T><<<dim3(n_tokens, 2 * nkv), 64, 0, s>>>(
      (const T*)kv, token_seq, token_pos, slots, block_table, (T*)k_pages, (T*)v_pages, nkv, D,
      max_pages, page);
  return gb_status();
}
GB_EXPORT int gb_kv_write_f32(const void* kv, const int* token_seq, const int* token_pos,
                              const int* slots, const int* block_table, void* k_pages,
                              void* v_pages, int n_tokens, int nkv, int D, int max_pages, int page,
                              cudaStream_t s) {
  return kv_write<float>(kv, token_seq, token_pos, slots, block_table, k_pages, v_pages, n_tokens,
                         nkv, D, max_pages, page, s);
}
GB_EXPORT int gb_kv_write_bf16(const void* kv, const int* token_seq, const int* token_pos,
                               const int* slots, const int* block_table, void* k_pages,
                               void* v_pages, int n_tokens, int nkv, int D, int max_pages, int page,
                               cudaStream_t s) {
  return kv_write<bf16>(kv, token_seq, token_pos, slots, block_table, k_pages, v_pages, n_tokens,
                        nkv, D, max_pages, page, s);
}
