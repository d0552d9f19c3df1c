// Thin wrappers over the sm_100a instructions that the tensor-memory kernels
// share: mbarriers with wall-clock-bounded waits, TMA tile loads (never with
// cluster multicast), tcgen05 MMA / commit / load / fences, and the shared-memory
// matrix descriptors of the 128-byte-swizzled tile layout that TMA writes.
#pragma once
#include <cuda.h>

#include <mutex>

#include "common.cuh"

#define TC_WAIT_LIMIT_NS 2000000000ull   // 2 s: far beyond any legitimate wait

// ---- PTX wrappers ------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(void* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(void* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(void* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P1;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P1;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// True in exactly one lane of a converged warp.  The compiler knows that the
// elected branch has one thread, which keeps the descriptors of the tcgen05
// instructions in it in uniform registers; a test of the lane index does not.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P1;\n\t"
      "elect.sync _|P1, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, P1;\n\t}"
      : "=r"(pred));
  return pred != 0;
}
// The state of the phase right now.  (try_wait may suspend the thread for a
// while when the phase is incomplete; a loop that watches several barriers must
// not.)
__device__ __forceinline__ bool mbar_test(void* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P1;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P1;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Waits for the phase with the given parity; false when the time limit expired
// or (where a flag is given) another role of the block has already given up.
__device__ __forceinline__ bool mbar_wait(void* bar, uint32_t parity, volatile int* abort_flag,
                                          unsigned long long limit_ns = TC_WAIT_LIMIT_NS) {
  if (mbar_try(bar, parity)) return true;
  const unsigned long long t0 = now_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try(bar, parity)) return true;
    if (abort_flag && *abort_flag) return mbar_try(bar, parity);
    if (now_ns() - t0 > limit_ns) return false;
  }
}
// The same for a whole converged warp: every lane polls and the lanes agree on
// the outcome by a vote, so that warp-wide instructions may follow either way.
// (One lane polling and broadcasting the result costs about 200 cycles more per
// wait than this: measured.)
__device__ __forceinline__ bool mbar_wait_warp(void* bar, uint32_t parity, volatile int* abort_flag,
                                               unsigned long long limit_ns = TC_WAIT_LIMIT_NS) {
  if (__all_sync(0xffffffffu, mbar_try(bar, parity))) return true;
  const unsigned long long t0 = now_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (__all_sync(0xffffffffu, mbar_try(bar, parity))) return true;
    const bool stop = (abort_flag && *abort_flag) || now_ns() - t0 > limit_ns;
    if (__any_sync(0xffffffffu, stop)) return __all_sync(0xffffffffu, mbar_try(bar, parity));
  }
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y,
                                            void* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Asks for a tensor map (a kernel parameter) to be brought into the TMA unit's
// descriptor cache, so that the first copy through it does not wait for it.
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(void* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same three for a converged warp: every lane executes the statement and
// the instruction is predicated on the elected lane, so that the descriptors are
// computed in warp-uniform code (the shape CUTLASS gives its issue loops).
// elect.sync with the full mask elects the same lane every time, which
// tcgen05.commit needs: it tracks the operations of the executing thread.
__device__ __forceinline__ void tc_commit_w(void* bar) {
  asm volatile(
      "{\n\t.reg .pred e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(
          smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tc_mma_w(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// A in tensor memory (lane = row, two bf16 of K a column), B through a descriptor
__device__ __forceinline__ void tc_mma_ta_w(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Four products of one 64-element slice of K in one statement, for a converged
// warp: one election, then the four instructions (and, where a barrier is given,
// a commit) predicated on the elected lane.  A burst written as separate elected
// statements pays for an election per instruction (about 29 cycles each,
// measured), and a branch that only one lane enters costs some hundred cycles to
// enter and leave; this form issues at under ten cycles an instruction.
// A from shared memory: the descriptors advance by a_step and b_step (in
// descriptor units of 16 bytes) per product.
template <bool COMMIT>
__device__ __forceinline__ void tc_mma_burst4_w(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                                uint32_t a_step, uint32_t b_step, uint32_t idesc,
                                                uint32_t first_accumulates, void* bar) {
  const uint64_t as = a_step, bs = b_step;
  asm volatile(
      "{\n\t.reg .pred e, p, c;\n\t.reg .b64 da, db;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "setp.ne.b32 c, %8, 0;\n\t"
      "and.pred c, c, e;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %5, p;\n\t"
      "setp.eq.b32 p, 0, 0;\n\t"
      "add.u64 da, %1, %3;\n\t"
      "add.u64 db, %2, %4;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t"
      "add.u64 da, da, %3;\n\t"
      "add.u64 db, db, %4;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t"
      "add.u64 da, da, %3;\n\t"
      "add.u64 db, db, %4;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t"
      "@c tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%7];\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "l"(as), "l"(bs), "r"(idesc), "r"(first_accumulates),
      "r"(COMMIT ? smem_u32(bar) : 0u), "r"(COMMIT ? 1u : 0u)
      : "memory");
}
// A from tensor memory: its address advances by 8 columns per product (16 bf16).
template <bool COMMIT>
__device__ __forceinline__ void tc_mma_ta_burst4_w(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                                   uint32_t b_step, uint32_t idesc,
                                                   uint32_t first_accumulates, void* bar) {
  const uint64_t bs = b_step;
  asm volatile(
      "{\n\t.reg .pred e, p, c;\n\t.reg .b32 ta;\n\t.reg .b64 db;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "setp.ne.b32 c, %7, 0;\n\t"
      "and.pred c, c, e;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %4, p;\n\t"
      "setp.eq.b32 p, 0, 0;\n\t"
      "add.u32 ta, %1, 8;\n\t"
      "add.u64 db, %2, %3;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %4, p;\n\t"
      "add.u32 ta, ta, 8;\n\t"
      "add.u64 db, db, %3;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %4, p;\n\t"
      "add.u32 ta, ta, 8;\n\t"
      "add.u64 db, db, %3;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %4, p;\n\t"
      "@c tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%6];\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "l"(bs), "r"(idesc), "r"(first_accumulates),
      "r"(COMMIT ? smem_u32(bar) : 0u), "r"(COMMIT ? 1u : 0u)
      : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns (the caller waits with tc_wait_ld)
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
               : "r"(taddr)
               : "memory");
}
// 32 lanes x 64 consecutive 32-bit columns (the caller waits with tc_wait_ld)
__device__ __forceinline__ void tc_ld64(uint32_t taddr, uint32_t (&v)[64]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31]), "=r"(v[32]), "=r"(v[33]), "=r"(v[34]), "=r"(v[35]), "=r"(v[36]), "=r"(v[37]), "=r"(v[38]), "=r"(v[39]), "=r"(v[40]), "=r"(v[41]), "=r"(v[42]), "=r"(v[43]), "=r"(v[44]), "=r"(v[45]), "=r"(v[46]), "=r"(v[47]), "=r"(v[48]), "=r"(v[49]), "=r"(v[50]), "=r"(v[51]), "=r"(v[52]), "=r"(v[53]), "=r"(v[54]), "=r"(v[55]), "=r"(v[56]), "=r"(v[57]), "=r"(v[58]), "=r"(v[59]), "=r"(v[60]), "=r"(v[61]), "=r"(v[62]), "=r"(v[63])
               : "r"(taddr)
               : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns, registers to tensor memory (the
// caller waits with tc_wait_st)
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
               :
               : "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
               : "memory");
}
__device__ __forceinline__ void tc_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major operand tile in shared memory, rows of 64 bf16 (128 bytes) under the
// 128-byte swizzle: groups of 8 rows are 1024 bytes apart (stride byte offset),
// the leading byte offset is unused for swizzled K-major layouts, descriptor
// version 1 (sm_100), layout type 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}


// ---- host: tensor maps ----------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn tc_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

// A bf16 matrix [rows, cols] with `pitch_bytes` between rows (a multiple of 16),
// read in boxes of box_rows x box_cols elements (box_cols * 2 <= 128 bytes) under
// the 128-byte swizzle; elements outside the matrix read as zero.
static inline int tc_make_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                                 uint64_t pitch_bytes, int box_rows, int box_cols) {
  EncodeTiledFn fn = tc_encode_fn();
  if (!fn) return GB_ERR_UNSUPPORTED;
  if ((pitch_bytes & 15) || (((uintptr_t)base) & 15)) return GB_ERR_BAD_ARG;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)pitch_bytes};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : GB_ERR_BAD_ARG;
}
