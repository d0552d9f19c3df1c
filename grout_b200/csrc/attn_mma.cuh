// Shared pieces of the bf16 attention kernels: asynchronous 16-byte copies into
// padded shared-memory tiles, ldmatrix fragment loads, and one step of the
// online-softmax recurrence for a warp that owns 16 query rows.
//
// Tiles are stored [row][D] with a row pitch of D + 8 elements: the pitch in
// 16-byte chunks is odd, so the eight rows that one ldmatrix phase touches fall
// into eight different bank groups for every head size that is a multiple of 16.
//
// The recurrence is the usual one (running maximum m, running sum l, rescaled
// accumulator), with scores kept in the log2 domain: p = 2^(s*c - m*c), c =
// scale * log2(e), as the reference's fmha kernels do (src/kernels.rs:1195-1291).
// Probabilities are rounded to bf16 for the P.V product (the reference rounds
// them to f16, src/kernels.rs:1282) while l sums the unrounded values.
#pragma once
#include "common.cuh"

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int sz = pred ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Where element (row, col) of a key or value tile lies in shared memory.
// PaddedTile: rows of D + 8 elements, written by 16-byte asynchronous copies.
// Swizzled128Tile: what TMA writes for boxes of ROWS x 64 elements under the
// 128-byte swizzle, one box per 64 columns, the boxes one after the other (each
// box 1024-byte aligned): the 16-byte chunk c of row r sits at chunk c ^ (r % 8).
// Both keep the eight rows of one ldmatrix phase in eight different bank groups.
template <int D>
struct PaddedTile {
  __device__ __forceinline__ static int off(int row, int col) { return row * (D + 8) + col; }
};
template <int ROWS>
struct Swizzled128Tile {
  __device__ __forceinline__ static int off(int row, int col) {
    return (col >> 6) * (ROWS * 64) + row * 64 + ((((col & 63) >> 3) ^ (row & 7)) << 3) + (col & 7);
  }
};

// The state of one warp's 16 query rows: this lane holds rows g = lane/4 and
// g + 8, and of every 8-wide group of columns the pair 2t, 2t+1 (t = lane%4).
template <int DT>  // head_dim = 16 * DT
struct WarpAttn {
  static constexpr int D = 16 * DT;
  static constexpr int LD = D + 8;  // row pitch of shared tiles, in elements
  uint32_t q[DT][4];                // A fragments of the 16 x D query tile
  float o[2 * DT][4];               // 16 x D accumulator
  float m[2], l[2];                 // running max (already times c) and this lane's share of l

  __device__ __forceinline__ void init() {
#pragma unroll
    for (int i = 0; i < 2 * DT; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
    m[0] = m[1] = -INFINITY;
    l[0] = l[1] = 0.f;
  }

  // q_tile: 16 rows of pitch LD in shared memory
  __device__ __forceinline__ void load_q(const bf16* q_tile) {
    const int lane = threadIdx.x & 31;
    const int row = (lane & 7) + ((lane >> 3) & 1) * 8, col = (lane >> 4) * 8;
#pragma unroll
    for (int k = 0; k < DT; ++k) ldmatrix_x4(q[k], q_tile + row * LD + k * 16 + col);
  }

  // One tile of NKEYS keys (a multiple of 16) held in shared memory as k_tile and
  // v_tile [NKEYS][LD].  Key index of tile row r is key0 + r.  Row `g` of this
  // lane sees keys in [lo[0], hi[0]], row g + 8 keys in [lo[1], hi[1]].
  template <int NKEYS, bool MASK>
  __device__ __forceinline__ void tile(const bf16* k_tile, const bf16* v_tile, int key0,
                                       const int (&lo)[2], const int (&hi)[2], float c) {
    tile<NKEYS, MASK>(k_tile, v_tile, key0, lo, hi, c, [] {});
  }

  // The same with `between()` called once the scores are computed, that is when k_tile has
  // been read for the last time and before v_tile is read for the first: a caller that
  // pipelines its copies refills the key buffer and waits for the values there.
  // L says where an element of a tile lies; the NKEYS keys are the tiles' rows row0 ..
  // row0 + NKEYS - 1 (row0 a multiple of 8).
  template <int NKEYS, bool MASK, typename L = PaddedTile<16 * DT>, typename F>
  __device__ __forceinline__ void tile(const bf16* k_tile, const bf16* v_tile, int key0,
                                       const int (&lo)[2], const int (&hi)[2], float c, F&& between,
                                       int row0 = 0) {
    const int lane = threadIdx.x & 31, t = lane & 3;
    constexpr int NT = NKEYS / 8;
    float s[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
    // S = Q K^T
    {
      const int krow = (lane & 7) + (lane >> 4) * 8, kcol = ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int k = 0; k < DT; ++k) {
#pragma unroll
        for (int j = 0; j < NT; j += 2) {
          uint32_t b[4];
          ldmatrix_x4(b, k_tile + L::off(row0 + j * 8 + krow, k * 16 + kcol));
          mma_16816(s[j], q[k], b[0], b[1]);
          mma_16816(s[j + 1], q[k], b[2], b[3]);
        }
      }
    }
    between();
    // scale into the log2 domain, mask, row maxima
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < NT; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        float v = s[j][e] * c;
        if (MASK) {
          const int key = key0 + j * 8 + t * 2 + (e & 1);
          if (key < lo[r] || key > hi[r]) v = -INFINITY;
        }
        s[j][e] = v;
        mx[r] = fmaxf(mx[r], v);
      }
    }
    float corr[2], base[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m[r], mx[r]);
      base[r] = (m_new == -INFINITY) ? 0.f : m_new;  // a row that has seen no key yet
      corr[r] = (m[r] == -INFINITY) ? 0.f : exp2f(m[r] - base[r]);
      m[r] = m_new;
      l[r] *= corr[r];
    }
#pragma unroll
    for (int i = 0; i < 2 * DT; ++i) {
      o[i][0] *= corr[0];
      o[i][1] *= corr[0];
      o[i][2] *= corr[1];
      o[i][3] *= corr[1];
    }
    // P = 2^(s - m), O += P V
    const int vrow = (lane & 7) + ((lane >> 3) & 1) * 8, vcol = (lane >> 4) * 8;
#pragma unroll
    for (int kk = 0; kk < NKEYS / 16; ++kk) {
      uint32_t p[4];
      float e0[4], e1[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        e0[e] = exp2f(s[2 * kk][e] - base[e >> 1]);
        e1[e] = exp2f(s[2 * kk + 1][e] - base[e >> 1]);
      }
      l[0] += e0[0] + e0[1] + e1[0] + e1[1];
      l[1] += e0[2] + e0[3] + e1[2] + e1[3];
      p[0] = pack_bf16(e0[0], e0[1]);
      p[1] = pack_bf16(e0[2], e0[3]);
      p[2] = pack_bf16(e1[0], e1[1]);
      p[3] = pack_bf16(e1[2], e1[3]);
#pragma unroll
      for (int i = 0; i < DT; ++i) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, v_tile + L::off(row0 + kk * 16 + vrow, i * 16 + vcol));
        mma_16816(o[2 * i], p, b[0], b[1]);
        mma_16816(o[2 * i + 1], p, b[2], b[3]);
      }
    }
  }

  // Sums l over the four lanes that share a row.
  __device__ __forceinline__ void finish_l() {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
  }
};
