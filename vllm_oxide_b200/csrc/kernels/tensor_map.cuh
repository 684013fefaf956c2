// Tensor maps (TMA descriptors) for row-major bfloat16 matrices, and the device-side copy that uses them.
//
// A matrix [rows, cols] (cols a multiple of 64) is described as a three-dimensional tensor
// (64 columns, rows, cols/64 column slices), and a box (64, box_rows, box_slices) is what ONE
// cp.async.bulk.tensor instruction copies into shared memory: slice after slice, each slice box_rows rows
// of 128 bytes in the 128-byte swizzled layout (the 16-byte chunk c of row r sits at chunk position
// c ^ (r % 8)).  One instruction per tile matters: issuing a copy costs the issuing thread a few hundred
// cycles whatever its size, so many small boxes starve the pipeline.  Rows and slices of the box outside
// the matrix arrive as zeros, so ragged edges need no special case.  The innermost coordinate of every copy
// is 0, which satisfies the copy engine's 16-byte alignment rule.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace vob {

#define VOB_ERR_TIMEOUT 32
// A kernel whose bounded wait runs out also says which kernel it is: its source file defines VOB_TIMEOUT_WHERE
// (one of the bits below) before it includes this header.
#define VOB_WHERE_GEMM_SKINNY 0x100
#define VOB_WHERE_GEMM_TC5 0x200
#define VOB_WHERE_ATTENTION_DECODE 0x400
#define VOB_WHERE_ATTENTION_PREFILL 0x800
#define VOB_WHERE_ATTENTION_PREFILL_TC5 0x1000
#ifndef VOB_TIMEOUT_WHERE
#define VOB_TIMEOUT_WHERE 0
#endif
#define VOB_ERR_TIMEOUT_BITS (VOB_ERR_TIMEOUT | VOB_TIMEOUT_WHERE)

constexpr unsigned MBAR_SPIN_LIMIT = 1u << 22;   // tries before a wait on an mbarrier gives up

// The limit that the pipeline waits (mbar_wait) use: MBAR_SPIN_LIMIT, unless a test has shortened it through its source
// file's setter to see a wait run out.  One copy per source file.  The drain at a kernel's end, which waits for copies
// that are already on their way, always uses MBAR_SPIN_LIMIT itself: no block leaves with a copy in flight.
static __device__ unsigned vob_wait_limit = MBAR_SPIN_LIMIT;
// For the same tests: non-zero makes a kernel's producer issue none of its copies, so that what waits for them waits
// for something that never comes (a try on an mbarrier may itself block for microseconds, long enough for a real copy
// to land, so a short limit alone does not make a wait run out).  Nothing is then in flight when the block leaves.
static __device__ unsigned vob_test_withhold_copies = 0;

// Host side of a source file's setter: tries 0 restores the default limit.
static inline int set_wait_limit(unsigned tries, unsigned withhold_copies) {
  const unsigned v = tries ? tries : MBAR_SPIN_LIMIT;
  cudaError_t e = cudaMemcpyToSymbol(vob_wait_limit, &v, sizeof(v));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(vob_test_withhold_copies, &withhold_copies, sizeof(withhold_copies));
  return (int)e;
}

__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
  unsigned ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// False when the wait ran out (or another thread of the block gave up before).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity, volatile int* abort_flag, int* err) {
  if (mbar_try_wait(bar, parity)) return true;      // the common case costs no read of the limit
  const unsigned limit = vob_wait_limit;
  for (unsigned i = 1; i < limit; ++i) {
    if (*abort_flag) return false;
    if (mbar_try_wait(bar, parity)) return true;
  }
  *abort_flag = 1;
  atomicOr(err, VOB_ERR_TIMEOUT_BITS);
  return false;
}

constexpr int TMA_BOX_COLS = 64;   // 128 bytes of bfloat16: the widest box the 128-byte swizzle allows

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int col, int row, uint64_t* bar) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
  const unsigned mbar = (unsigned)__cvta_generic_to_shared(bar);
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
               ::"r"(dst), "l"(map), "r"(col), "r"(row), "r"(mbar) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
  const unsigned mbar = (unsigned)__cvta_generic_to_shared(bar);
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(mbar) : "memory");
}
// A tile from shared memory to global memory (the tile's layout as a load would have written it).  The copies of a
// thread form groups: commit, then wait until the group's shared memory has been read before it is reused or the block
// ends.  What the copies wrote is visible to other kernels when this one has ended.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* smem_src, int c0, int c1, int c2) {
  const unsigned src = (unsigned)__cvta_generic_to_shared(smem_src);
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];\n"
               ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory"); }
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];\n" ::"l"(map) : "memory");
}
// Byte offset of (row, 16-byte chunk) inside a swizzled box whose base is 1024-byte aligned.
__device__ __forceinline__ int swizzled_offset(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

}  // namespace vob
