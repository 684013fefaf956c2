// Causal grouped-query attention over the paged cache, for any mix of prompt portions and
// single decoded tokens: the plain kernel.  It serves the true 32-bit path and every size the
// faster kernels refuse.
//
// One block per (token, query head).  The keys a query may read are lo..pos, with
// pos the query's position and lo = max(0, pos - window + 1) (0 without a window).  They are
// walked in tiles of 32 ALIGNED TO ABSOLUTE POSITIONS; tile j belongs to warp j % 4.  Each
// warp keeps a running maximum, sum and weighted value sum in float (an online softmax), and
// the four warps are merged in a fixed order.  So the sequence of float operations for a
// query depends only on (lo, pos) and on the cache's contents at those positions: not on how
// the tokens were cut into steps, not on what else is in the batch, not on which pages hold
// the keys.  Scale 1/sqrt(hd) is applied to the score as the reference does
// (vllm-oxide, crates/vllm-oxide/src/models/qwen3.rs:204-209); query head h reads key/value
// head h / (nh/kvh).
#include "common.cuh"

namespace vob {

constexpr int ATT_WARPS = 4;
constexpr int ATT_MAXD = 16;  // value dims per lane: hd <= 512

template <typename T>
__device__ __forceinline__ float dot_row(const float* q, const T* k, int hd);

template <>
__device__ __forceinline__ float dot_row<float>(const float* q, const float* k, int hd) {
  float s = 0.f;
  const float4* k4 = reinterpret_cast<const float4*>(k);
  for (int i = 0; i < hd / 4; ++i) {
    const float4 v = k4[i];
    s += q[4 * i] * v.x; s += q[4 * i + 1] * v.y; s += q[4 * i + 2] * v.z; s += q[4 * i + 3] * v.w;
  }
  return s;
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* q, const __nv_bfloat16* k,
                                                         int hd) {
  float s = 0.f;
  const uint4* k8 = reinterpret_cast<const uint4*>(k);
  for (int i = 0; i < hd / 8; ++i) {
    const uint4 raw = k8[i];
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h2[j]);
      s += q[8 * i + 2 * j] * f.x;
      s += q[8 * i + 2 * j + 1] * f.y;
    }
  }
  return s;
}

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
paged_attention_generic_kernel(const T* q, long q_stride, T* out,
                               const T* kcache, const T* vcache,
                               const int* __restrict__ block_tables, int table_stride,
                               const int* __restrict__ token_req, const int* __restrict__ positions,
                               const int* __restrict__ skip_single_cu_q, int nh, int kvh, int hd, int block_size,
                               int window, float scale, long num_pages, int* err) {
  extern __shared__ float smem[];
  float* qs = smem;                        // [hd]
  float* accs = smem + hd;                 // [ATT_WARPS][hd]
  __shared__ float ms[ATT_WARPS], ls[ATT_WARPS];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const int req = token_req[t];
  if (req < 0) return;
  if (skip_single_cu_q && skip_single_cu_q[req + 1] - skip_single_cu_q[req] == 1) return;  // the decode kernel's
  const int pos = positions[t];
  const int kh = h / (nh / kvh);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const T* qrow = q + (size_t)t * q_stride + (size_t)h * hd;
  for (int i = threadIdx.x; i < hd; i += blockDim.x) qs[i] = to_f<T>(qrow[i]);
  __syncthreads();
  const int* table = block_tables + (size_t)req * table_stride;

  float m = -INFINITY, l = 0.f;
  float acc[ATT_MAXD];
#pragma unroll
  for (int j = 0; j < ATT_MAXD; ++j) acc[j] = 0.f;

  for (int tile = lo / 32 + ((warp - (lo / 32) % ATT_WARPS + ATT_WARPS) % ATT_WARPS); tile <= pos / 32; tile += ATT_WARPS) {
    const int key = tile * 32 + lane;
    const bool valid = key >= lo && key <= pos;
    long row = -1;  // element offset of this key's row for kv head kh
    if (valid) {
      const int page = table[key / block_size];
      if (page < 0 || page >= num_pages) atomicOr(err, VOB_ERR_PAGE);
      else row = (((long)page * kvh + kh) * block_size + key % block_size) * (long)hd;
    }
    float s = -INFINITY;
    if (row >= 0) s = dot_row<T>(qs, kcache + row, hd) * scale;
    const float m_new = fmaxf(m, warp_max(s));
    const float p = (row >= 0) ? expf(s - m_new) : 0.f;
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int j = 0; j < ATT_MAXD; ++j) acc[j] *= corr;
    for (int kk = 0; kk < 32; ++kk) {
      const long rk = __shfl_sync(0xffffffffu, row, kk);
      if (rk < 0) continue;
      const float pk = __shfl_sync(0xffffffffu, p, kk);
      const T* vrow = vcache + rk;
#pragma unroll
      for (int j = 0; j < ATT_MAXD; ++j) {
        const int d = lane + 32 * j;
        if (d < hd) acc[j] += pk * to_f<T>(vrow[d]);
      }
    }
    m = m_new;
  }
  if (lane == 0) { ms[warp] = m; ls[warp] = l; }
#pragma unroll
  for (int j = 0; j < ATT_MAXD; ++j) {
    const int d = lane + 32 * j;
    if (d < hd) accs[warp * hd + d] = acc[j];
  }
  __syncthreads();
  float mm = -INFINITY;
#pragma unroll
  for (int w = 0; w < ATT_WARPS; ++w) mm = fmaxf(mm, ms[w]);
  float f[ATT_WARPS], lt = 0.f;
#pragma unroll
  for (int w = 0; w < ATT_WARPS; ++w) {
    f[w] = (ms[w] == -INFINITY) ? 0.f : expf(ms[w] - mm);
    lt += ls[w] * f[w];
  }
  T* orow = out + (size_t)t * nh * hd + (size_t)h * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) o += accs[w * hd + d] * f[w];
    orow[d] = from_f<T>(lt > 0.f ? o / lt : 0.f);
  }
}

}  // namespace vob

using namespace vob;

// q: rows of q_stride elements, head h at h*hd; out [T, nh*hd]; caches [num_pages, kvh, block_size, hd];
// block_tables [B, table_stride]; token_req [T] (-1: padding); positions [T].
VOB_API int vob_paged_attention_generic(const void* q, long q_stride, void* out, const void* kcache, const void* vcache,
                                        const int* block_tables, int table_stride, const int* token_req,
                                        const int* positions, const int* skip_single_cu_q, int T, int nh, int kvh, int hd,
                                        int block_size,
                                        int window, float scale, long num_pages, int dtype, int* err,
                                        cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd <= 0 || hd % 16 || hd > 512 || kvh <= 0 || nh % kvh || block_size <= 0) return VOB_UNSUPPORTED;
  dim3 grid(T, nh);
  const size_t smem = (size_t)(1 + ATT_WARPS) * hd * sizeof(float);
  if (dtype == VOB_F32)
    return launch_kernel(paged_attention_generic_kernel<float>, grid, ATT_WARPS * 32, smem, stream, (const float*)q, q_stride,
                         (float*)out, (const float*)kcache, (const float*)vcache, block_tables, table_stride, token_req,
                         positions, skip_single_cu_q, nh, kvh, hd, block_size, window, scale, num_pages, err);
  if (dtype == VOB_BF16)
    return launch_kernel(paged_attention_generic_kernel<__nv_bfloat16>, grid, ATT_WARPS * 32, smem, stream,
                         (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, (const __nv_bfloat16*)kcache,
                         (const __nv_bfloat16*)vcache, block_tables, table_stride, token_req, positions, skip_single_cu_q,
                         nh, kvh, hd, block_size, window, scale, num_pages, err);
  return VOB_BAD_ARGUMENT;
}
