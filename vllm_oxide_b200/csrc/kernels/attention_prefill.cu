// Causal attention for prompt portions over the paged cache in bfloat16 (tensor cores).
//
// A request's portion of n tokens at positions ctx-n .. ctx-1 attends to everything the cache holds
// for it (earlier portions, prefix-cache hits, and the portion itself, which was written first).
// Grid (row block, kv head, request), 128 threads.  The "rows" of a request are its (token, query
// head of the group) pairs, token-major; a block owns 64 consecutive rows, 16 per warp, so the
// heads of a group share every key and value brought in.  Keys are walked in tiles of 64 from
// the lowest position any row of the block may read to the highest, copied into shared memory with
// cp.async in 3 stages; each warp masks by its rows' own positions (causal, and the window if any)
// and runs the online softmax of attention_mma.cuh.  Requests that bring exactly one token are
// skipped (the decode kernel takes them).  Compiled once per head size (-DVOB_HD).
#include "attention_mma.cuh"

namespace vob {

constexpr int PF_TILE = 64;
constexpr int PF_WARPS = 4;
constexpr int PF_ROWS = PF_WARPS * 16;
constexpr int PF_STAGES = HD <= 128 ? 3 : 2;
constexpr int PF_STAGE_BYTES = 2 * PF_TILE * ROW_BYTES;

__global__ void __launch_bounds__(PF_WARPS * 32)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, long q_stride, __nv_bfloat16* __restrict__ out,
                         const __nv_bfloat16* __restrict__ kcache, const __nv_bfloat16* __restrict__ vcache,
                         const int* __restrict__ block_tables, int table_stride, const int* __restrict__ cu_q,
                         const int* __restrict__ context_lens, int nh, int kvh, int block_size, int window, float scale,
                         long num_pages, int* err) {
  extern __shared__ __align__(16) char smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int kh = blockIdx.y, b = blockIdx.z;
  const int t0 = cu_q[b];
  const int n = cu_q[b + 1] - t0;
  if (n <= 1) return;                                   // nothing, or a decoding request
  const int G = nh / kvh;
  const int total_rows = n * G;
  const int row0 = blockIdx.x * PF_ROWS;
  if (row0 >= total_rows) return;
  const int ctx = context_lens[b];
  const int first_pos = ctx - n;                        // position of the portion's first token
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int* table = block_tables + (size_t)b * table_stride;

  // this thread's two rows: token and head, position, validity
  int rpos[2], rtok[2], rhead[2];
  bool rvalid[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = row0 + warp * 16 + g + 8 * h;
    rvalid[h] = row < total_rows;
    rtok[h] = rvalid[h] ? row / G : 0;
    rhead[h] = kh * G + (rvalid[h] ? row % G : 0);
    rpos[h] = first_pos + rtok[h];
  }
  uint32_t qf[KSTEPS][4];
  {
    const __nv_bfloat16* q0 = q + (size_t)(t0 + rtok[0]) * q_stride + (size_t)rhead[0] * HD;
    const __nv_bfloat16* q1 = q + (size_t)(t0 + rtok[1]) * q_stride + (size_t)rhead[1] * HD;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      const int d = ks * 16 + tq * 2;
      qf[ks][0] = rvalid[0] ? *reinterpret_cast<const uint32_t*>(q0 + d) : 0u;
      qf[ks][1] = rvalid[1] ? *reinterpret_cast<const uint32_t*>(q1 + d) : 0u;
      qf[ks][2] = rvalid[0] ? *reinterpret_cast<const uint32_t*>(q0 + d + 8) : 0u;
      qf[ks][3] = rvalid[1] ? *reinterpret_cast<const uint32_t*>(q1 + d + 8) : 0u;
    }
  }
  // key range of the block and of this warp
  const int last_row = min(row0 + PF_ROWS, total_rows) - 1;
  const int blk_pos_lo = first_pos + row0 / G, blk_pos_hi = first_pos + last_row / G;
  const int key_lo = window > 0 ? max(0, blk_pos_lo - window + 1) : 0;
  const int key_end = blk_pos_hi + 1;
  const int w_first = min(row0 + warp * 16, last_row), w_last = min(row0 + warp * 16 + 15, last_row);
  const int w_pos_lo = first_pos + w_first / G, w_pos_hi = first_pos + w_last / G;
  const int w_key_lo = window > 0 ? max(0, w_pos_lo - window + 1) : 0;
  const bool warp_active = row0 + warp * 16 < total_rows;

  WarpSoftmax st;
  st.clear();
  const float sc = scale * LOG2E;
  const int start = key_lo / PF_TILE * PF_TILE;
  const int n_tiles = (key_end - start + PF_TILE - 1) / PF_TILE;
  int pages[PF_TILE / RUN_KEYS];
#pragma unroll
  for (int s = 0; s < PF_STAGES - 1; ++s) {
    if (s < n_tiles) {
      tile_pages<PF_TILE>(pages, table, block_size, start + s * PF_TILE, key_lo, key_end);
      load_kv_tile<PF_TILE, PF_WARPS * 32>(smem + s * PF_STAGE_BYTES, kcache, vcache, pages, block_size, kvh, kh,
                                           start + s * PF_TILE, key_lo, key_end, num_pages, err);
    }
    cp_async_commit();
  }
  if (PF_STAGES - 1 < n_tiles) tile_pages<PF_TILE>(pages, table, block_size, start + (PF_STAGES - 1) * PF_TILE, key_lo, key_end);
  for (int it = 0; it < n_tiles; ++it) {
    const int nxt = it + PF_STAGES - 1;
    if (nxt < n_tiles) {
      load_kv_tile<PF_TILE, PF_WARPS * 32>(smem + (nxt % PF_STAGES) * PF_STAGE_BYTES, kcache, vcache, pages, block_size, kvh,
                                           kh, start + nxt * PF_TILE, key_lo, key_end, num_pages, err);
      if (nxt + 1 < n_tiles) tile_pages<PF_TILE>(pages, table, block_size, start + (nxt + 1) * PF_TILE, key_lo, key_end);
    }
    cp_async_commit();
    cp_async_wait<PF_STAGES - 1>();
    __syncthreads();
    const char* stage = smem + (it % PF_STAGES) * PF_STAGE_BYTES;
    const int tile_k0 = start + it * PF_TILE;
    if (warp_active) {
#pragma unroll
      for (int sub = 0; sub < PF_TILE / 16; ++sub) {
        const int k0 = tile_k0 + sub * 16;
        if (k0 > w_pos_hi || k0 + 15 < w_key_lo) continue;       // nothing here for this warp's rows
        float s[2][4];
        qk_16keys(qf, stage + sub * 16 * ROW_BYTES, lane, s);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int h = e >> 1;
            const int key = k0 + i * 8 + tq * 2 + (e & 1);
            bool ok = rvalid[h] && key <= rpos[h];
            if (window > 0) ok = ok && key > rpos[h] - window;
            s[i][e] = ok ? s[i][e] * sc : -INFINITY;
          }
        }
        softmax_pv_16keys(st, s, stage + PF_TILE * ROW_BYTES + sub * 16 * ROW_BYTES, lane);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 1);
    st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (!rvalid[h]) continue;
    const float inv = st.l[h] > 0.f ? 1.f / st.l[h] : 0.f;
    __nv_bfloat16* orow = out + (size_t)(t0 + rtok[h]) * nh * HD + (size_t)rhead[h] * HD + tq * 2;
#pragma unroll
    for (int j = 0; j < DTILES; ++j)
      *reinterpret_cast<__nv_bfloat162*>(orow + j * 8) = __floats2bfloat162_rn(st.o[j][2 * h] * inv, st.o[j][2 * h + 1] * inv);
  }
}

}  // namespace vob

using namespace vob;

// max_q: the most tokens any request brings in this step (sizes the grid).
VOB_API int vob_attention_prefill(const void* q, long q_stride, void* out, const void* kcache, const void* vcache,
                                  const int* block_tables, int table_stride, const int* cu_q, const int* context_lens,
                                  int num_requests, int max_q, int nh, int kvh, int block_size, int window, float scale,
                                  long num_pages, int* err, cudaStream_t stream) {
  if (num_requests <= 0 || max_q <= 1) return 0;
  if (kvh <= 0 || nh % kvh || block_size <= 0 || kvh > 65535 || num_requests > 65535) return VOB_UNSUPPORTED;
  static bool configured = false;
  const int smem = PF_STAGES * PF_STAGE_BYTES;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const long rows = (long)max_q * (nh / kvh);
  dim3 grid((unsigned)((rows + PF_ROWS - 1) / PF_ROWS), kvh, num_requests);
  return launch_kernel(attention_prefill_kernel, grid, PF_WARPS * 32, smem, stream, (const __nv_bfloat16*)q, q_stride,
                       (__nv_bfloat16*)out, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, block_tables,
                       table_stride, cu_q, context_lens, nh, kvh, block_size, window, scale, num_pages, err);
}
