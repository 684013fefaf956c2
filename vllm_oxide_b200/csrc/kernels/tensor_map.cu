// Host side of tensor maps: encodes a CUtensorMap for a row-major bfloat16 matrix.
// The driver's encoder is looked up at run time, so the library links against the runtime only.
#include "tensor_map.cuh"

namespace vob {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}
}  // namespace vob

using namespace vob;

// out_map: 128 bytes, 64-byte aligned, on the host.  The box is [box_rows, 64 columns], 128-byte swizzle.
// Needs a 16-byte aligned base, a row stride that is a multiple of 8 elements, box_rows <= 256.
VOB_API int vob_tensor_map_bf16_2d(void* out_map, const void* base, long rows, long cols, long row_stride, int box_rows) {
  if (!out_map || !base || rows <= 0 || cols <= 0 || box_rows <= 0 || box_rows > 256) return VOB_BAD_ARGUMENT;
  if (((uintptr_t)base) % 16 || (row_stride * 2) % 16 || ((uintptr_t)out_map) % 64) return VOB_UNSUPPORTED;
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return VOB_UNSUPPORTED;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
  const cuuint32_t box[2] = {(cuuint32_t)TMA_BOX_COLS, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = fn((CUtensorMap*)out_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : VOB_BAD_ARGUMENT;
}

// The same matrix as (64 columns, rows, cols/64 slices) with box (64, box_rows, box_slices): one copy brings
// box_slices column slices of box_rows rows each.  Needs cols to be a multiple of 64.
VOB_API int vob_tensor_map_bf16_sliced(void* out_map, const void* base, long rows, long cols, long row_stride, int box_rows,
                                       int box_slices) {
  if (!out_map || !base || rows <= 0 || cols <= 0 || box_rows <= 0 || box_rows > 256 || box_slices <= 0 || box_slices > 256)
    return VOB_BAD_ARGUMENT;
  if (cols % TMA_BOX_COLS || ((uintptr_t)base) % 16 || (row_stride * 2) % 16 || ((uintptr_t)out_map) % 64) return VOB_UNSUPPORTED;
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return VOB_UNSUPPORTED;
  const cuuint64_t dims[3] = {(cuuint64_t)TMA_BOX_COLS, (cuuint64_t)rows, (cuuint64_t)(cols / TMA_BOX_COLS)};
  const cuuint64_t strides[2] = {(cuuint64_t)row_stride * 2, (cuuint64_t)TMA_BOX_COLS * 2};
  const cuuint32_t box[3] = {(cuuint32_t)TMA_BOX_COLS, (cuuint32_t)box_rows, (cuuint32_t)box_slices};
  const cuuint32_t elem[3] = {1, 1, 1};
  CUresult r = fn((CUtensorMap*)out_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : VOB_BAD_ARGUMENT;
}

// Token rows of `heads` heads of `head_dim` elements each (head h of token t at base + t * token_stride + h * head_dim),
// seen as (head_dim, heads, tokens) with box (64 columns, box_heads, box_tokens): one copy brings a 64-column slice of
// box_heads heads for box_tokens tokens, as rows of 128 bytes in the order (token, head), 128-byte swizzled.
VOB_API int vob_tensor_map_bf16_heads(void* out_map, const void* base, long tokens, int heads, int head_dim, long token_stride,
                                      int box_heads, int box_tokens) {
  if (!out_map || !base || tokens <= 0 || heads <= 0 || head_dim <= 0 || box_heads <= 0 || box_heads > 256 || box_tokens <= 0 ||
      box_tokens > 256)
    return VOB_BAD_ARGUMENT;
  if (head_dim % TMA_BOX_COLS || ((uintptr_t)base) % 16 || (token_stride * 2) % 16 || ((uintptr_t)out_map) % 64) return VOB_UNSUPPORTED;
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return VOB_UNSUPPORTED;
  const cuuint64_t dims[3] = {(cuuint64_t)head_dim, (cuuint64_t)heads, (cuuint64_t)tokens};
  const cuuint64_t strides[2] = {(cuuint64_t)head_dim * 2, (cuuint64_t)token_stride * 2};
  const cuuint32_t box[3] = {(cuuint32_t)TMA_BOX_COLS, (cuuint32_t)box_heads, (cuuint32_t)box_tokens};
  const cuuint32_t elem[3] = {1, 1, 1};
  CUresult r = fn((CUtensorMap*)out_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : VOB_BAD_ARGUMENT;
}
