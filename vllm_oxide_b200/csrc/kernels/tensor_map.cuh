// Tensor maps (TMA descriptors) for row-major bfloat16 matrices, and the device-side copy that uses them.
//
// A map describes a matrix [rows, cols] with a row stride and a box [box_rows, 64 columns] that one
// cp.async.bulk.tensor instruction copies into shared memory in the 128-byte swizzled layout: row r of
// the box occupies 128 bytes, and its 16-byte chunk c sits at chunk position c ^ (r % 8).  Elements of
// the box outside the matrix arrive as zeros, so ragged edges need no special case.  The innermost
// coordinate of every copy in this package is a multiple of 64 columns (128 bytes), as the copy engine
// requires 16-byte alignment there.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace vob {

constexpr int TMA_BOX_COLS = 64;   // 128 bytes of bfloat16: the widest box the 128-byte swizzle allows

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int col, int row, uint64_t* bar) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
  const unsigned mbar = (unsigned)__cvta_generic_to_shared(bar);
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
               ::"r"(dst), "l"(map), "r"(col), "r"(row), "r"(mbar) : "memory");
}
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];\n" ::"l"(map) : "memory");
}
// Byte offset of (row, 16-byte chunk) inside a swizzled box whose base is 1024-byte aligned.
__device__ __forceinline__ int swizzled_offset(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

}  // namespace vob
