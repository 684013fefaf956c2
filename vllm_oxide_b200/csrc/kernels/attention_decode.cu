// Decode attention over the paged cache in bfloat16: one query token per request, keys split
// over several blocks, the query heads of a key/value head processed together.
//
// Grid (split, kv head, request), 128 threads.  A block owns a contiguous range of the keys the
// query may read (lo..pos, lo = max(0, pos - window + 1)), walks it in tiles of 64 keys brought
// into shared memory with cp.async (3 stages; every cache row is found through the block table,
// so any page size works), and each of its 4 warps takes 16 keys of a tile: Q.K^T and P.V run on
// tensor cores (m16n8k16) with the group's query heads as the 16 rows, the softmax is online in
// float.  The warps are merged through shared memory; with several splits the block writes a
// normalised partial result and its log-sum-exp to scratch memory, and a second kernel merges the
// splits.  Requests that bring more than one token are skipped (the prefill kernel takes them).
// Compiled once per head size (-DVOB_HD).
#define VOB_TIMEOUT_WHERE 0x400
#include "attention_mma.cuh"

namespace vob {

constexpr int DEC_TILE = 64;   // keys per tile
constexpr int DEC_WARPS = 4;
constexpr int DEC_STAGES = HD <= 128 ? 3 : 2;
constexpr int DEC_STAGE_BYTES = 2 * DEC_TILE * ROW_BYTES;   // K tile, then V tile

__global__ void __launch_bounds__(DEC_WARPS * 32)
attention_decode_kernel(const __nv_bfloat16* q, long q_stride, __nv_bfloat16* out,
                        const __nv_bfloat16* kcache, const __nv_bfloat16* vcache,
                        const int* __restrict__ block_tables, int table_stride, const int* __restrict__ cu_q,
                        const int* __restrict__ context_lens, int nh, int kvh, int block_size, int window, float scale,
                        long num_pages, float* part_o, float* part_lse, int* err) {
  extern __shared__ __align__(16) char smem[];
  pdl_launch_dependents();
  const int split = blockIdx.x, num_splits = gridDim.x, kh = blockIdx.y, b = blockIdx.z;
  const int t = cu_q[b];
  const int t_next = cu_q[b + 1], context = context_lens[b];   // the step's index arrays: written before the step
  pdl_wait();                                                   // the query, and this token's key and value, are not
  if (t_next - t != 1) return;                         // not a decoding request
  const int G = nh / kvh;
  const int pos = context - 1;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  // the key range in tiles of 64 from lo rounded down to a multiple of 16 (the copies work in runs of 16
  // keys); split s takes tiles [s*n/S, (s+1)*n/S): within one tile of each other
  const int lo16 = lo & ~15;
  const int all_tiles = (pos + 1 - lo16 + DEC_TILE - 1) / DEC_TILE;
  const int tile_begin = (int)((long)split * all_tiles / num_splits);
  const int tile_end = (int)((long)(split + 1) * all_tiles / num_splits);
  const int start = lo16 + tile_begin * DEC_TILE;
  const int end = min(pos + 1, lo16 + tile_end * DEC_TILE);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int* table = block_tables + (size_t)b * table_stride;

  // the group's query heads as rows 0..G-1 of a 16-row tile (other rows zero), in A-fragment layout
  uint32_t qf[KSTEPS][4];
  {
    const __nv_bfloat16* qrow0 = q + (size_t)t * q_stride + (size_t)(kh * G + g) * HD;
    const __nv_bfloat16* qrow1 = qrow0 + (size_t)8 * HD;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      const int d = ks * 16 + tq * 2;
      qf[ks][0] = g < G ? *reinterpret_cast<const uint32_t*>(qrow0 + d) : 0u;
      qf[ks][1] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qrow1 + d) : 0u;
      qf[ks][2] = g < G ? *reinterpret_cast<const uint32_t*>(qrow0 + d + 8) : 0u;
      qf[ks][3] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qrow1 + d + 8) : 0u;
    }
  }
  WarpSoftmax st;
  st.clear();
  const float sc = scale * LOG2E;
  const int n_tiles = start < end ? (end - start + DEC_TILE - 1) / DEC_TILE : 0;
  int pages[DEC_TILE / RUN_KEYS];
#pragma unroll
  for (int s = 0; s < DEC_STAGES - 1; ++s) {
    if (s < n_tiles) {
      tile_pages<DEC_TILE>(pages, table, block_size, start + s * DEC_TILE, lo, end);
      load_kv_tile<DEC_TILE, DEC_WARPS * 32>(smem + s * DEC_STAGE_BYTES, kcache, vcache, pages, block_size, kvh, kh,
                                             start + s * DEC_TILE, lo, end, num_pages, err);
    }
    cp_async_commit();
  }
  if (DEC_STAGES - 1 < n_tiles) tile_pages<DEC_TILE>(pages, table, block_size, start + (DEC_STAGES - 1) * DEC_TILE, lo, end);
  for (int it = 0; it < n_tiles; ++it) {
    const int nxt = it + DEC_STAGES - 1;
    if (nxt < n_tiles) {
      load_kv_tile<DEC_TILE, DEC_WARPS * 32>(smem + (nxt % DEC_STAGES) * DEC_STAGE_BYTES, kcache, vcache, pages, block_size,
                                             kvh, kh, start + nxt * DEC_TILE, lo, end, num_pages, err);
      // the pages of the tile after that: looked up now, used in the next round
      if (nxt + 1 < n_tiles) tile_pages<DEC_TILE>(pages, table, block_size, start + (nxt + 1) * DEC_TILE, lo, end);
    }
    cp_async_commit();
    cp_async_wait<DEC_STAGES - 1>();
    __syncthreads();
    const char* stage = smem + (it % DEC_STAGES) * DEC_STAGE_BYTES;
    const int k0 = start + it * DEC_TILE + warp * 16;
    if (k0 < end) {
      float s[2][4];
      qk_16keys(qf, stage + warp * 16 * ROW_BYTES, lane, s);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int key = k0 + i * 8 + tq * 2;
        const bool ok0 = key >= lo && key < end, ok1 = key + 1 >= lo && key + 1 < end;
        s[i][0] = ok0 ? s[i][0] * sc : -INFINITY;
        s[i][1] = ok1 ? s[i][1] * sc : -INFINITY;
        s[i][2] = ok0 ? s[i][2] * sc : -INFINITY;
        s[i][3] = ok1 ? s[i][3] * sc : -INFINITY;
      }
      softmax_pv_16keys(st, s, stage + DEC_TILE * ROW_BYTES + warp * 16 * ROW_BYTES, lane);
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();
  // merge the warps: shared memory now holds, per warp, m[16], l[16] and o[16][HD]
  float* wm = reinterpret_cast<float*>(smem);                 // [DEC_WARPS][16]
  float* wl = wm + DEC_WARPS * 16;                            // [DEC_WARPS][16]
  float* wo = wl + DEC_WARPS * 16;                            // [DEC_WARPS][16][HD]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 1);
    st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 2);
  }
  if (tq == 0) {
    wm[warp * 16 + g] = st.m[0]; wm[warp * 16 + g + 8] = st.m[1];
    wl[warp * 16 + g] = st.l[0]; wl[warp * 16 + g + 8] = st.l[1];
  }
#pragma unroll
  for (int j = 0; j < DTILES; ++j) {
    float* r0 = wo + ((size_t)warp * 16 + g) * HD + j * 8 + tq * 2;
    float* r1 = wo + ((size_t)warp * 16 + g + 8) * HD + j * 8 + tq * 2;
    r0[0] = st.o[j][0]; r0[1] = st.o[j][1];
    r1[0] = st.o[j][2]; r1[1] = st.o[j][3];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * HD; idx += DEC_WARPS * 32) {
    const int r = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, wm[w * 16 + r]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float f = wm[w * 16 + r] == -INFINITY ? 0.f : fast_exp2(wm[w * 16 + r] - M);
      L += wl[w * 16 + r] * f;
      O += wo[((size_t)w * 16 + r) * HD + d] * f;
    }
    const float val = L > 0.f ? O / L : 0.f;
    const int head = kh * G + r;
    if (num_splits == 1) {
      out[(size_t)t * nh * HD + (size_t)head * HD + d] = __float2bfloat16_rn(val);
    } else {
      const size_t p = ((size_t)b * nh + head) * num_splits + split;
      part_o[p * HD + d] = val;
      if (d == 0) part_lse[p] = L > 0.f ? M + log2f(L) : -INFINITY;
    }
  }
}

#if VOB_HD % 64 == 0
// ---- the same kernel with the keys and values brought in by TMA ------------------------------------------
// cp.async moves about 16 bytes per clock and SM on this GPU, the copy engine about twice that, so head sizes
// that are a multiple of 64 (one or more 128-byte swizzled column slices) take this kernel.  A fifth warp is the
// producer: its lanes look the pages of eight tiles up at once, a chunk ahead (a look-up is a load with a long
// latency, and a producer that needs one per tile cannot run ahead of it), and one thread issues one copy of K and
// one of V per tile when pages hold a multiple of 64 keys (a tile then lies in one page), else one per run of 16
// keys; a copy brings all column slices at once.  An mbarrier per stage counts the bytes in, a second one the four
// consumer warps out.  Every wait is bounded.  With 2 to 8 splits the blocks of a (request, kv head) are launched as
// a thread-block cluster and merge their results through each other's shared memory; with more they write partial
// results to scratch memory for the merge kernel.  tmK / tmV describe a cache plane as a matrix [pages * kv_heads * block_size, HD] in
// column slices, with boxes of `box_keys` (64 or 16) rows.
constexpr int DT_SLICES = HD / 64;
constexpr int DT_TILE_BYTES = DT_SLICES * DEC_TILE * 128;       // one of K or V
constexpr int DT_STAGE_BYTES = 2 * DT_TILE_BYTES;
constexpr int DT_STAGES = HD <= 128 ? 3 : 2;
constexpr int DT_THREADS = (DEC_WARPS + 1) * 32;

__global__ void __launch_bounds__(DT_THREADS)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                            const __nv_bfloat16* q, long q_stride, __nv_bfloat16* out,
                            const int* __restrict__ block_tables, int table_stride, const int* __restrict__ cu_q,
                            const int* __restrict__ context_lens, int nh, int kvh, int block_size, int window, float scale,
                            long num_pages, float* part_o, float* part_lse,
                            int box_keys, int cluster, int* err) {
  extern __shared__ __align__(1024) char smem_raw[];
  char* smem = reinterpret_cast<char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int MERGE_BYTES = (2 * DEC_WARPS * 16 + DEC_WARPS * 16 * HD) * 4;
  constexpr int FINAL_BYTES = (16 * HD + 16) * 4;
  constexpr int DATA_BYTES = DT_STAGES * DT_STAGE_BYTES > MERGE_BYTES + FINAL_BYTES ? DT_STAGES * DT_STAGE_BYTES : MERGE_BYTES + FINAL_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + DATA_BYTES);
  uint64_t* empty = full + DT_STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + DT_STAGES);
  pdl_launch_dependents();
  const int split = blockIdx.x, num_splits = gridDim.x, kh = blockIdx.y, b = blockIdx.z;
  const int t = cu_q[b];
  const int t_next = cu_q[b + 1], context = context_lens[b];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < DT_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], DEC_WARPS); }
    *abort_flag = 0;
    tma_prefetch_map(&tmK);
    tma_prefetch_map(&tmV);
  }
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  __syncthreads();
  // The step's index arrays, the block tables and the keys and values before this step's token were written
  // before this step's kernels began; the kernels of this step write this token's query, key and value only.
  // So the producer waits for the kernels before this one only when it comes to the tile that holds the new key,
  // and the consumers wait before they read the query: the older tiles stream in while those kernels still run.
  if (t_next - t != 1) { pdl_wait(); return; }         // not a decoding request (uniform for the block)
  const int G = nh / kvh;
  const int pos = context - 1;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int lo16 = lo & ~(box_keys - 1);               // tiles start on a box boundary
  const int all_tiles = (pos + 1 - lo16 + DEC_TILE - 1) / DEC_TILE;
  const int tile_begin = (int)((long)split * all_tiles / num_splits);
  const int tile_end = (int)((long)(split + 1) * all_tiles / num_splits);
  const int start = lo16 + tile_begin * DEC_TILE;
  const int end = min(pos + 1, lo16 + tile_end * DEC_TILE);
  const int n_tiles = start < end ? (end - start + DEC_TILE - 1) / DEC_TILE : 0;
  const int* table = block_tables + (size_t)b * table_stride;
  WarpSoftmax st;
  st.clear();

  if (warp == DEC_WARPS) {
    // ------------------------------------------------ producer: lane 0 issues, all lanes look pages up
    {
      WarpPages wp;
      bool ok = true, waited = false;
      int it = 0;
      for (; it < n_tiles; ++it) {
        const int s = it % DT_STAGES;
        wp.advance(table, block_size, start, it, lane, lo, end);
        int pg[4];
#pragma unroll
        for (int run = 0; run < 4; ++run) pg[run] = wp.page(it, run);
        if (lane == 0) {
          if (it >= DT_STAGES) ok = mbar_wait(&empty[s], (unsigned)(((it / DT_STAGES) - 1) & 1), abort_flag, err);
          if (ok) {
            const int tile_start = start + it * DEC_TILE;
            if (!waited && tile_start + DEC_TILE > pos) { pdl_wait(); waited = true; }
            mbar_expect_tx(&full[s], (unsigned)DT_STAGE_BYTES);
            char* kt = smem + s * DT_STAGE_BYTES;
            if (box_keys == DEC_TILE) {
              // the tile lies in one page: one copy of K, one of V (any run that is wanted names the page)
              const int page = pg[0] != PAGE_NONE ? pg[0] : (pg[1] != PAGE_NONE ? pg[1] : (pg[2] != PAGE_NONE ? pg[2] : pg[3]));
              const bool page_ok = page >= 0 && page < num_pages;
              if (!page_ok && page != PAGE_NONE) atomicOr(err, VOB_ERR_PAGE);
              const int row = page_ok ? (page * kvh + kh) * block_size + tile_start % block_size : 0;
              tma_load_3d(kt, &tmK, 0, row, 0, &full[s]);
              tma_load_3d(kt + DT_TILE_BYTES, &tmV, 0, row, 0, &full[s]);
            } else {
#pragma unroll
              for (int run = 0; run < 4; ++run) {
                const bool page_ok = pg[run] >= 0 && pg[run] < num_pages;
                if (!page_ok && pg[run] != PAGE_NONE) atomicOr(err, VOB_ERR_PAGE);
                // a run nobody will read is filled from row 0 of the plane: finite values that the mask zeroes
                const int key0 = tile_start + run * RUN_KEYS;
                const int row = page_ok ? (pg[run] * kvh + kh) * block_size + key0 % block_size : 0;
                // a 16-row box writes its slices 16 rows apart, the tile keeps them DEC_TILE rows apart: a copy per slice
#pragma unroll
                for (int c = 0; c < DT_SLICES; ++c) {
                  tma_load_3d(kt + c * DEC_TILE * 128 + run * RUN_KEYS * 128, &tmK, 0, row, c, &full[s]);
                  tma_load_3d(kt + DT_TILE_BYTES + c * DEC_TILE * 128 + run * RUN_KEYS * 128, &tmV, 0, row, c, &full[s]);
                }
              }
            }
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
      }
      if (lane == 0) {
        const int first = it > DT_STAGES ? it - DT_STAGES : 0;     // copies in flight must land before the block exits
        for (int j = first; j < it; ++j) {
          bool done = false;
          for (unsigned i = 0; i < MBAR_SPIN_LIMIT && !done; ++i) done = mbar_try_wait(&full[j % DT_STAGES], (unsigned)((j / DT_STAGES) & 1));
          if (!done) atomicOr(err, VOB_ERR_TIMEOUT_BITS);
        }
      }
    }
  } else {
    // ------------------------------------------------ consumers: warp w takes keys 16w..16w+15 of every tile
    pdl_wait();
    const int g = lane >> 2, tq = lane & 3;
    uint32_t qf[KSTEPS][4];
    {
      const __nv_bfloat16* qrow0 = q + (size_t)t * q_stride + (size_t)(kh * G + g) * HD;
      const __nv_bfloat16* qrow1 = qrow0 + (size_t)8 * HD;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        const int d = ks * 16 + tq * 2;
        qf[ks][0] = g < G ? *reinterpret_cast<const uint32_t*>(qrow0 + d) : 0u;
        qf[ks][1] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qrow1 + d) : 0u;
        qf[ks][2] = g < G ? *reinterpret_cast<const uint32_t*>(qrow0 + d + 8) : 0u;
        qf[ks][3] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qrow1 + d + 8) : 0u;
      }
    }
    const float sc = scale * LOG2E;
    for (int it = 0; it < n_tiles; ++it) {
      const int s = it % DT_STAGES;
      bool ok = mbar_wait(&full[s], (unsigned)((it / DT_STAGES) & 1), abort_flag, err);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const char* kt = smem + s * DT_STAGE_BYTES;
      const int k0 = start + it * DEC_TILE + warp * 16;
      if (k0 < end && k0 + 16 > lo) {
        float sv[2][4];
        qk_16keys_swizzled<DEC_TILE>(qf, kt, warp * 16, lane, sv);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int key = k0 + i * 8 + tq * 2;
          const bool ok0 = key >= lo && key < end, ok1 = key + 1 >= lo && key + 1 < end;
          sv[i][0] = ok0 ? sv[i][0] * sc : -INFINITY;
          sv[i][1] = ok1 ? sv[i][1] * sc : -INFINITY;
          sv[i][2] = ok0 ? sv[i][2] * sc : -INFINITY;
          sv[i][3] = ok1 ? sv[i][3] * sc : -INFINITY;
        }
        softmax_pv_16keys_swizzled<DEC_TILE>(st, sv, kt + DT_TILE_BYTES, warp * 16, lane);
      }
      // ordinary loads of the stage before the copy engine's next write to it: a proxy fence, then the release
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
  }
  pdl_wait();             // (a no-op for threads that have waited) nothing is written before the kernels before are done
  __syncthreads();        // every stage has been read (or given up): the merge may reuse the memory
  const bool aborted = *abort_flag != 0;
  if (aborted && !cluster) return;
  float* wm = reinterpret_cast<float*>(smem);                 // [DEC_WARPS][16]
  float* wl = wm + DEC_WARPS * 16;
  float* wo = wl + DEC_WARPS * 16;                            // [DEC_WARPS][16][HD]
  float* fo = reinterpret_cast<float*>(smem + MERGE_BYTES);   // [16][HD] this block's result, for the other blocks of a cluster
  float* fl = fo + 16 * HD;                                   // [16] its log-sum-exp
  if (warp < DEC_WARPS) {
    const int g = lane >> 2, tq = lane & 3;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 1);
      st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 2);
    }
    if (tq == 0) {
      wm[warp * 16 + g] = st.m[0]; wm[warp * 16 + g + 8] = st.m[1];
      wl[warp * 16 + g] = st.l[0]; wl[warp * 16 + g + 8] = st.l[1];
    }
#pragma unroll
    for (int j = 0; j < DTILES; ++j) {
      float* r0 = wo + ((size_t)warp * 16 + g) * HD + j * 8 + tq * 2;
      float* r1 = wo + ((size_t)warp * 16 + g + 8) * HD + j * 8 + tq * 2;
      r0[0] = st.o[j][0]; r0[1] = st.o[j][1];
      r1[0] = st.o[j][2]; r1[1] = st.o[j][3];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * HD; idx += DT_THREADS) {
    const int r = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, wm[w * 16 + r]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float f = wm[w * 16 + r] == -INFINITY ? 0.f : fast_exp2(wm[w * 16 + r] - M);
      L += wl[w * 16 + r] * f;
      O += wo[((size_t)w * 16 + r) * HD + d] * f;
    }
    const float val = L > 0.f ? O / L : 0.f;
    const float lse = (L > 0.f && !aborted) ? M + log2f(L) : -INFINITY;
    const int head = kh * G + r;
    if (num_splits == 1) {
      out[(size_t)t * nh * HD + (size_t)head * HD + d] = __float2bfloat16_rn(val);
    } else if (cluster) {
      fo[idx] = val;
      if (d == 0) fl[r] = lse;
    } else {
      const size_t p = ((size_t)b * nh + head) * num_splits + split;
      part_o[p * HD + d] = val;
      if (d == 0) part_lse[p] = lse;
    }
  }
  if (num_splits == 1 || !cluster) return;
  // The blocks of a (request, kv head) form a thread-block cluster: each reads the others' results from their shared
  // memory and merges a share of the outputs (weights 2^(lse - max lse), in the order of the splits).  Every block
  // of the cluster comes to both barriers, also one that gave up (its log-sum-exp is -inf: weight zero).
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
  {
    const unsigned fo_addr = smem_addr(fo), fl_addr = smem_addr(fl);
    for (int idx = split * DT_THREADS + threadIdx.x; idx < G * HD; idx += num_splits * DT_THREADS) {
      const int r = idx / HD;
      // every block's log-sum-exp and value for this output: all the loads from the other blocks' shared memory are
      // issued before the first result is used (one after the other they cost a round trip across the cluster each,
      // sixteen of them with eight splits: more than a microsecond)
      float lse[8], v[8];
#pragma unroll
      for (int sp = 0; sp < 8; ++sp) {
        lse[sp] = -INFINITY;
        v[sp] = 0.f;
        if (sp < num_splits) {
          unsigned ra, rb;
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(ra) : "r"(fl_addr + r * 4), "r"(sp));
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(rb) : "r"(fo_addr + idx * 4), "r"(sp));
          asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(lse[sp]) : "r"(ra) : "memory");
          asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v[sp]) : "r"(rb) : "memory");
        }
      }
      float M = -INFINITY;
#pragma unroll
      for (int sp = 0; sp < 8; ++sp) M = fmaxf(M, lse[sp]);
      float W = 0.f, O = 0.f;
#pragma unroll
      for (int sp = 0; sp < 8; ++sp) {        // in the order of the splits; a split that is not there weighs nothing
        const float w = lse[sp] == -INFINITY ? 0.f : fast_exp2(lse[sp] - M);
        W += w;
        O += w * v[sp];
      }
      out[(size_t)t * nh * HD + (size_t)(kh * G) * HD + idx] = __float2bfloat16_rn(W > 0.f ? O / W : 0.f);
    }
  }
  // nobody may leave while another block still reads its shared memory
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

// ---- many decoding requests, one split each ---------------------------------------------------------------------------
// With more (request, kv head) pairs than blocks fit the GPU, a block of the kernel above lives for a dozen tiles, and a
// good part of that is its start: the look-up of its pages, the first copies, nothing to compute on yet.  Here the blocks
// are persistent instead.  Block i begins with pair i and takes its further pairs from a counter in device memory (so
// that requests of very different lengths spread as evenly as blocks given out by the hardware would), and its producer
// warp runs AHEAD across pairs: the ring of stages never drains between two pairs, so the pages of the next pair are
// looked up and its first tiles are on their way while the consumer warps still work on the pair before.  The producer
// tells the consumers which pair a tile opens through a small queue in shared memory, written before the tile's
// mbarrier is armed; after its last pair it sends an entry that says "no more" the same way.  The four warps' results of a
// pair meet in a buffer of their own (not in the ring, which is busy), between two barriers of the consumer warps alone.
// Same tiles, same products, same order of additions as the kernel above with one split: the same bits.
//
// The counter is the caller's: two words of device memory, zero before the first launch; the last block to leave sets
// them back to zero.  Launches that may overlap in time (two streams) need counters of their own; the engine gives every
// attention layer one.  The producer takes from it only after it has waited for the kernels before this one, and a
// kernel is done only when each of its blocks has; so a launch of an earlier step of the same stream has left the
// counter at zero by then.
constexpr int DI_MERGE_FLOATS(int G) { return 2 * DEC_WARPS * 16 + DEC_WARPS * G * HD; }
constexpr int DI_DRAW_AHEAD = 2;                          // tiles before a pair's last at which the next pair is drawn
constexpr int DI_QUEUE = 8;                               // entries; the producer is at most DT_STAGES + 1 pairs ahead

__global__ void __launch_bounds__(DT_THREADS)
attention_decode_tma_items_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                                  const __nv_bfloat16* q, long q_stride, __nv_bfloat16* out,
                                  const int* __restrict__ block_tables, int table_stride, const int* __restrict__ cu_q,
                                  const int* __restrict__ context_lens, int num_requests, int nh, int kvh, int block_size,
                                  int window, float scale, long num_pages, int box_keys, unsigned* pairs_taken, int* err) {
  // pairs_taken[0]: pairs given out beyond the first of each block; [1]: blocks that have left
  extern __shared__ __align__(1024) char smem_raw[];
  char* smem = reinterpret_cast<char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int RING_BYTES = DT_STAGES * DT_STAGE_BYTES;
  const int G = nh / kvh;
  float* wm = reinterpret_cast<float*>(smem + RING_BYTES);    // [DEC_WARPS][16]
  float* wl = wm + DEC_WARPS * 16;
  float* wo = wl + DEC_WARPS * 16;                            // [DEC_WARPS][G][HD]
  int4* queue = reinterpret_cast<int4*>(wo + DEC_WARPS * G * HD);   // (pair or -1, its token's row, its position, -)
  uint64_t* full = reinterpret_cast<uint64_t*>(queue + DI_QUEUE);
  uint64_t* empty = full + DT_STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + DT_STAGES);
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < DT_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], DEC_WARPS); }
    *abort_flag = 0;
    tma_prefetch_map(&tmK);
    tma_prefetch_map(&tmV);
  }
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  __syncthreads();
  const int num_items = num_requests * kvh;

  if (warp == DEC_WARPS) {
    // ------------------------------------------------ producer: lane 0 issues, all lanes look pages up
    bool ok = true, waited = false;                   // `waited`: this warp has waited for the kernels before this one
    long ring = 0;                                    // stages armed so far, over all pairs: stage = ring % DT_STAGES
    int pairs = 0;                                    // pairs announced to the consumers
    int item = blockIdx.x;
    while (ok && item < num_items) {
      // The pair after this one is drawn a few tiles before this one's last, so that the counter's answer is back when
      // this pair's tiles are out, yet no block holds a pair long before it can begin it (a block that has not waited
      // yet draws after its tiles: the counter is this launch's only after the launches before it are done).
      int next = -1;
      bool drawn = false;
      const int b = item / kvh, kh = item % kvh;
      const int t = cu_q[b];
      if (cu_q[b + 1] - t == 1) {                     // a decoding request (the others are the prefill kernel's)
        const int pos = context_lens[b] - 1;
        const int lo = window > 0 ? max(0, pos - window + 1) : 0;
        const int start = lo & ~(box_keys - 1);
        const int end = pos + 1;
        const int n_tiles = (end - start + DEC_TILE - 1) / DEC_TILE;
        const int* table = block_tables + (size_t)b * table_stride;
        WarpPages wp;
        for (int it = 0; it < n_tiles; ++it, ++ring) {
          const int s = (int)(ring % DT_STAGES);
          wp.advance(table, block_size, start, it, lane, lo, end);
          int pg[4];
#pragma unroll
          for (int run = 0; run < 4; ++run) pg[run] = wp.page(it, run);
          if (waited && !drawn && it + DI_DRAW_AHEAD >= n_tiles) {
            if (lane == 0) next = (int)min((unsigned)num_items, gridDim.x + atomicAdd(&pairs_taken[0], 1u));
            drawn = true;
          }
          if (lane == 0) {
            if (ring >= DT_STAGES) ok = mbar_wait(&empty[s], (unsigned)(((ring / DT_STAGES) - 1) & 1), abort_flag, err);
            if (ok) {
              const int tile_start = start + it * DEC_TILE;
              // only the tile that holds this step's key waits for the kernels before this one (once for the block)
              if (!waited && tile_start + DEC_TILE > pos) { pdl_wait(); waited = true; }
              if (it == 0) queue[pairs % DI_QUEUE] = make_int4(item, t, pos, 0);   // before the arrival below releases it
              mbar_expect_tx(&full[s], (unsigned)DT_STAGE_BYTES);
              char* kt = smem + s * DT_STAGE_BYTES;
              if (box_keys == DEC_TILE) {
                const int page = pg[0] != PAGE_NONE ? pg[0] : (pg[1] != PAGE_NONE ? pg[1] : (pg[2] != PAGE_NONE ? pg[2] : pg[3]));
                const bool page_ok = page >= 0 && page < num_pages;
                if (!page_ok && page != PAGE_NONE) atomicOr(err, VOB_ERR_PAGE);
                const int row = page_ok ? (page * kvh + kh) * block_size + tile_start % block_size : 0;
                tma_load_3d(kt, &tmK, 0, row, 0, &full[s]);
                tma_load_3d(kt + DT_TILE_BYTES, &tmV, 0, row, 0, &full[s]);
              } else {
#pragma unroll
                for (int run = 0; run < 4; ++run) {
                  const bool page_ok = pg[run] >= 0 && pg[run] < num_pages;
                  if (!page_ok && pg[run] != PAGE_NONE) atomicOr(err, VOB_ERR_PAGE);
                  const int key0 = tile_start + run * RUN_KEYS;
                  const int row = page_ok ? (pg[run] * kvh + kh) * block_size + key0 % block_size : 0;
#pragma unroll
                  for (int c = 0; c < DT_SLICES; ++c) {
                    tma_load_3d(kt + c * DEC_TILE * 128 + run * RUN_KEYS * 128, &tmK, 0, row, c, &full[s]);
                    tma_load_3d(kt + DT_TILE_BYTES + c * DEC_TILE * 128 + run * RUN_KEYS * 128, &tmV, 0, row, c, &full[s]);
                  }
                }
              }
            }
          }
          const int flags = __shfl_sync(0xffffffffu, (ok ? 1 : 0) | (waited ? 2 : 0), 0);
          ok = (flags & 1) != 0;
          waited = (flags & 2) != 0;
          if (!ok) break;
        }
        ++pairs;
      }
      if (!ok) break;
      if (!drawn && lane == 0) {
        if (!waited) pdl_wait();
        next = (int)min((unsigned)num_items, gridDim.x + atomicAdd(&pairs_taken[0], 1u));
      }
      waited = true;
      item = __shfl_sync(0xffffffffu, next, 0);
    }
    if (lane == 0) {
      if (ok) {                                       // "no more", in the stage the consumers wait on next
        const int s = (int)(ring % DT_STAGES);
        if (ring >= DT_STAGES) ok = mbar_wait(&empty[s], (unsigned)(((ring / DT_STAGES) - 1) & 1), abort_flag, err);
        if (ok) {
          queue[pairs % DI_QUEUE] = make_int4(-1, 0, 0, 0);
          mbar_arrive(&full[s]);
          ++ring;
        }
      }
      const long first = ring > DT_STAGES ? ring - DT_STAGES : 0;   // copies in flight must land before the block exits
      for (long j = first; j < ring; ++j) {
        bool done = false;
        for (unsigned i = 0; i < MBAR_SPIN_LIMIT && !done; ++i) done = mbar_try_wait(&full[j % DT_STAGES], (unsigned)((j / DT_STAGES) & 1));
        if (!done) atomicOr(err, VOB_ERR_TIMEOUT_BITS);
      }
    }
  } else {
    // ------------------------------------------------ consumers: warp w takes keys 16w..16w+15 of every tile
    // Every pair, and the entry that ends the list, takes a warp through the same two barriers, also a warp whose wait
    // ran out (it has raised the flag before it arrives); after the second barrier all four see the flag and leave.
    pdl_wait();
    const int g = lane >> 2, tq = lane & 3;
    const float sc = scale * LOG2E;
    long ring = 0;
    for (int pair = 0;; ++pair) {
      bool ok = mbar_wait(&full[ring % DT_STAGES], (unsigned)((ring / DT_STAGES) & 1), abort_flag, err);
      ok = __all_sync(0xffffffffu, ok);
      const int4 entry = ok ? queue[pair % DI_QUEUE] : make_int4(-1, 0, 0, 0);
      const bool more = entry.x >= 0;
      const int kh = more ? entry.x % kvh : 0, t = entry.y, pos = entry.z;
      const int lo = window > 0 ? max(0, pos - window + 1) : 0;
      const int start = lo & ~(box_keys - 1);
      const int end = pos + 1;
      const int n_tiles = more ? (end - start + DEC_TILE - 1) / DEC_TILE : 0;
      WarpSoftmax st;
      st.clear();
      if (more) {
        uint32_t qf[KSTEPS][4];
        const __nv_bfloat16* qrow0 = q + (size_t)t * q_stride + (size_t)(kh * G + g) * HD;
        const __nv_bfloat16* qrow1 = qrow0 + (size_t)8 * HD;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
          const int d = ks * 16 + tq * 2;
          qf[ks][0] = g < G ? *reinterpret_cast<const uint32_t*>(qrow0 + d) : 0u;
          qf[ks][1] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qrow1 + d) : 0u;
          qf[ks][2] = g < G ? *reinterpret_cast<const uint32_t*>(qrow0 + d + 8) : 0u;
          qf[ks][3] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qrow1 + d + 8) : 0u;
        }
        for (int it = 0; it < n_tiles; ++it, ++ring) {
          const int s = (int)(ring % DT_STAGES);
          if (it > 0) {
            ok = mbar_wait(&full[s], (unsigned)((ring / DT_STAGES) & 1), abort_flag, err);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
          }
          const char* kt = smem + s * DT_STAGE_BYTES;
          const int k0 = start + it * DEC_TILE + warp * 16;
          if (k0 < end && k0 + 16 > lo) {
            float sv[2][4];
            qk_16keys_swizzled<DEC_TILE>(qf, kt, warp * 16, lane, sv);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const int key = k0 + i * 8 + tq * 2;
              const bool ok0 = key >= lo && key < end, ok1 = key + 1 >= lo && key + 1 < end;
              sv[i][0] = ok0 ? sv[i][0] * sc : -INFINITY;
              sv[i][1] = ok1 ? sv[i][1] * sc : -INFINITY;
              sv[i][2] = ok0 ? sv[i][2] * sc : -INFINITY;
              sv[i][3] = ok1 ? sv[i][3] * sc : -INFINITY;
            }
            softmax_pv_16keys_swizzled<DEC_TILE>(st, sv, kt + DT_TILE_BYTES, warp * 16, lane);
          }
          asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(&empty[s]);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 1);
          st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 2);
        }
        if (tq == 0) {
          wm[warp * 16 + g] = st.m[0]; wm[warp * 16 + g + 8] = st.m[1];
          wl[warp * 16 + g] = st.l[0]; wl[warp * 16 + g + 8] = st.l[1];
        }
#pragma unroll
        for (int j = 0; j < DTILES; ++j) {
          if (g < G) {
            float* r0 = wo + ((size_t)warp * G + g) * HD + j * 8 + tq * 2;
            r0[0] = st.o[j][0]; r0[1] = st.o[j][1];
          }
          if (g + 8 < G) {
            float* r1 = wo + ((size_t)warp * G + g + 8) * HD + j * 8 + tq * 2;
            r1[0] = st.o[j][2]; r1[1] = st.o[j][3];
          }
        }
      }
      asm volatile("bar.sync 1, %0;\n" ::"n"(DEC_WARPS * 32) : "memory");
      const bool aborted = *abort_flag != 0;
      if (more && !aborted) {
        for (int idx = threadIdx.x; idx < G * HD; idx += DEC_WARPS * 32) {
          const int r = idx / HD, d = idx % HD;
          float M = -INFINITY;
#pragma unroll
          for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, wm[w * 16 + r]);
          float L = 0.f, O = 0.f;
#pragma unroll
          for (int w = 0; w < DEC_WARPS; ++w) {
            const float f = wm[w * 16 + r] == -INFINITY ? 0.f : fast_exp2(wm[w * 16 + r] - M);
            L += wl[w * 16 + r] * f;
            O += wo[((size_t)w * G + r) * HD + d] * f;
          }
          out[(size_t)t * nh * HD + (size_t)(kh * G + r) * HD + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
        }
      }
      asm volatile("bar.sync 1, %0;\n" ::"n"(DEC_WARPS * 32) : "memory");   // the buffer is free for the next pair
      if (!more || aborted) break;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {                             // the last block to leave makes the counter ready for the next launch
    __threadfence();
    if (atomicAdd(&pairs_taken[1], 1u) == gridDim.x - 1) {
      pairs_taken[0] = 0;
      pairs_taken[1] = 0;
      __threadfence();
    }
  }
}
#endif  // VOB_HD % 64 == 0

// Merges the splits of every (decoding request, head): weights 2^(lse - max lse).
__global__ void attention_decode_combine_kernel(const float* part_o, const float* part_lse,
                                                __nv_bfloat16* out, const int* __restrict__ cu_q, int nh,
                                                int num_splits) {
  pdl_launch_dependents();
  const int b = blockIdx.y, head = blockIdx.x;
  const int t = cu_q[b];
  const int t_next = cu_q[b + 1];
  pdl_wait();
  if (t_next - t != 1) return;
  const size_t base = ((size_t)b * nh + head) * num_splits;
  float M = -INFINITY;
  for (int s = 0; s < num_splits; ++s) M = fmaxf(M, part_lse[base + s]);
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float W = 0.f, O = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const float lse = part_lse[base + s];
      const float w = lse == -INFINITY ? 0.f : exp2f(lse - M);
      W += w;
      O += w * part_o[(base + s) * HD + d];
    }
    out[(size_t)t * nh * HD + (size_t)head * HD + d] = __float2bfloat16_rn(W > 0.f ? O / W : 0.f);
  }
}

}  // namespace vob

using namespace vob;

VOB_API int vob_attention_decode_head_dim() { return HD; }

// Programmatic dependent launch on (default) or off, for every kernel of this library.
VOB_API void vob_set_pdl(int on) { pdl_enabled() = on != 0; }

// Floats of scratch memory a launch with these sizes needs (0 with one split).
VOB_API long vob_attention_decode_scratch_floats(int num_requests, int nh, int num_splits) {
  return num_splits > 1 ? (long)num_requests * nh * num_splits * (HD + 1) : 0;
}

static bool g_decode_cluster_merge = true;
// Up to 8 splits merge through a thread-block cluster (default) or through scratch memory and a second kernel.
VOB_API void vob_attention_decode_cluster_merge(int on) { g_decode_cluster_merge = on != 0; }

static int attention_decode_launch(const void* map_k, const void* map_v, const void* q, long q_stride, void* out,
                                   const void* kcache, const void* vcache, const int* block_tables, int table_stride,
                                   const int* cu_q, const int* context_lens, int num_requests, int nh, int kvh,
                                   int block_size, int window, float scale, long num_pages, int num_splits, float* scratch,
                                   unsigned* pairs_counter, int* err, cudaStream_t stream) {
  if (num_requests <= 0) return 0;
  if (kvh <= 0 || nh % kvh || nh / kvh > 16 || block_size <= 0 || num_splits < 1 || num_splits > 65535) return VOB_UNSUPPORTED;
  static bool configured = false;
  const int merge_bytes = (2 * DEC_WARPS * 16 + DEC_WARPS * 16 * HD) * (int)sizeof(float);
  const int smem = DEC_STAGES * DEC_STAGE_BYTES > merge_bytes ? DEC_STAGES * DEC_STAGE_BYTES : merge_bytes;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  float* part_o = scratch;
  float* part_lse = scratch ? scratch + (size_t)num_requests * nh * num_splits * HD : nullptr;
  dim3 grid(num_splits, kvh, num_requests);
  int rc;
#if VOB_HD % 64 == 0
  if (map_k && map_v && block_size % 16 == 0) {
    static bool tma_configured = false;
    constexpr int MERGE = (2 * DEC_WARPS * 16 + DEC_WARPS * 16 * HD) * 4 + (16 * HD + 16) * 4;
    constexpr int DATA = DT_STAGES * DT_STAGE_BYTES > MERGE ? DT_STAGES * DT_STAGE_BYTES : MERGE;
    const int tma_smem = 1024 + DATA + 2 * DT_STAGES * 8 + 32;
    if (!tma_configured) {
      cudaError_t e = cudaFuncSetAttribute(attention_decode_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, tma_smem);
      if (e != cudaSuccess) return (int)e;
      tma_configured = true;
    }
    const int box_keys = block_size % DEC_TILE == 0 ? DEC_TILE : RUN_KEYS;
    // one split and more (request, kv head) pairs than blocks fit the GPU: persistent blocks, the producer ahead across pairs
    if (num_splits == 1 && pairs_counter) {
      const int G = nh / kvh;
      const int items_smem = 1024 + DT_STAGES * DT_STAGE_BYTES + DI_MERGE_FLOATS(G) * 4 + DI_QUEUE * 16 + 2 * DT_STAGES * 8 + 32;
      static int resident_of[17] = {0};      // blocks that fit the GPU at once, by heads per kv head (0: not asked yet)
      if (!resident_of[G]) {
        static int items_configured = 0;
        if (items_configured < items_smem) {
          cudaError_t e = cudaFuncSetAttribute(attention_decode_tma_items_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, items_smem);
          if (e != cudaSuccess) return (int)e;
          items_configured = items_smem;
        }
        int per_sm = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_decode_tma_items_kernel, DT_THREADS, items_smem);
        if (e != cudaSuccess) return (int)e;
        resident_of[G] = (per_sm > 0 ? per_sm : 1) * sm_count();
      }
      if ((long)num_requests * kvh > resident_of[G])
        return launch_kernel(attention_decode_tma_items_kernel, dim3(resident_of[G]), DT_THREADS, items_smem, stream,
                             *(const CUtensorMap*)map_k, *(const CUtensorMap*)map_v, (const __nv_bfloat16*)q, q_stride,
                             (__nv_bfloat16*)out, block_tables, table_stride, cu_q, context_lens, num_requests, nh, kvh,
                             block_size, window, scale, num_pages, box_keys, pairs_counter, err);
    }
    // up to 8 splits: the blocks of a (request, kv head) are a cluster and merge through shared memory
    if (num_splits > 1 && num_splits <= 8 && g_decode_cluster_merge)
      return launch_kernel_cluster(attention_decode_tma_kernel, grid, DT_THREADS, tma_smem, stream, (unsigned)num_splits,
                                   *(const CUtensorMap*)map_k, *(const CUtensorMap*)map_v, (const __nv_bfloat16*)q, q_stride,
                                   (__nv_bfloat16*)out, block_tables, table_stride, cu_q, context_lens, nh, kvh, block_size,
                                   window, scale, num_pages, part_o, part_lse, box_keys, 1, err);
    if (num_splits > 1 && !scratch) return VOB_BAD_ARGUMENT;
    rc = launch_kernel(attention_decode_tma_kernel, grid, DT_THREADS, tma_smem, stream, *(const CUtensorMap*)map_k,
                       *(const CUtensorMap*)map_v, (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, block_tables,
                       table_stride, cu_q, context_lens, nh, kvh, block_size, window, scale, num_pages, part_o, part_lse,
                       box_keys, 0, err);
    if (rc || num_splits == 1) return rc;
    return launch_kernel(attention_decode_combine_kernel, dim3(nh, num_requests), HD < 128 ? 64 : 128, 0, stream,
                         (const float*)part_o, (const float*)part_lse, (__nv_bfloat16*)out, cu_q, nh, num_splits);
  }
#endif
  if (num_splits > 1 && !scratch) return VOB_BAD_ARGUMENT;
  rc = launch_kernel(attention_decode_kernel, grid, DEC_WARPS * 32, smem, stream, (const __nv_bfloat16*)q, q_stride,
                         (__nv_bfloat16*)out, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, block_tables,
                         table_stride, cu_q, context_lens, nh, kvh, block_size, window, scale, num_pages, part_o, part_lse,
                         err);
  if (rc || num_splits == 1) return rc;
  return launch_kernel(attention_decode_combine_kernel, dim3(nh, num_requests), HD < 128 ? 64 : 128, 0, stream,
                       (const float*)part_o, (const float*)part_lse, (__nv_bfloat16*)out, cu_q, nh, num_splits);
}

// q rows of q_stride elements (head h at h*HD); out [T, nh*HD]; caches [num_pages, kvh, block_size, HD];
// block_tables [B, table_stride]; cu_q [B+1]; context_lens [B]; scratch: vob_attention_decode_scratch_floats.
VOB_API int vob_attention_decode(const void* q, long q_stride, void* out, const void* kcache, const void* vcache,
                                 const int* block_tables, int table_stride, const int* cu_q, const int* context_lens,
                                 int num_requests, int nh, int kvh, int block_size, int window, float scale,
                                 long num_pages, int num_splits, float* scratch, int* err, cudaStream_t stream) {
  return attention_decode_launch(nullptr, nullptr, q, q_stride, out, kcache, vcache, block_tables, table_stride, cu_q,
                                 context_lens, num_requests, nh, kvh, block_size, window, scale, num_pages, num_splits,
                                 scratch, nullptr, err, stream);
}

// The same with the caches also given as tensor maps (vob_tensor_map_bf16_sliced over [pages*kvh*block_size, HD] with
// boxes of vob_attention_decode_box_keys(block_size) rows and vob_attention_decode_box_slices(block_size) slices): head
// sizes that are a multiple of 64 then bring keys and values in by TMA.  Null maps fall back to cp.async.
// pairs_counter (may be null): two words of device memory, zero before the first call and left at zero by every call,
// not shared with a call that may run at the same time.  With it, one split and more (request, kv head) pairs than
// blocks fit the GPU run as persistent blocks that draw their pairs from it; without it, as one block per pair.
VOB_API int vob_attention_decode_tma(const void* map_k, const void* map_v, const void* q, long q_stride, void* out,
                                     const void* kcache, const void* vcache, const int* block_tables, int table_stride,
                                     const int* cu_q, const int* context_lens, int num_requests, int nh, int kvh,
                                     int block_size, int window, float scale, long num_pages, int num_splits,
                                     float* scratch, unsigned* pairs_counter, int* err, cudaStream_t stream) {
  return attention_decode_launch(map_k, map_v, q, q_stride, out, kcache, vcache, block_tables, table_stride, cu_q,
                                 context_lens, num_requests, nh, kvh, block_size, window, scale, num_pages, num_splits,
                                 scratch, pairs_counter, err, stream);
}

VOB_API int vob_attention_decode_has_tma() { return VOB_HD % 64 == 0 ? 1 : 0; }
VOB_API int vob_attention_decode_box_keys(int block_size) { return block_size % DEC_TILE == 0 ? DEC_TILE : RUN_KEYS; }
VOB_API int vob_attention_decode_box_slices(int block_size) { return block_size % DEC_TILE == 0 ? HD / 64 : 1; }

// ------------------------------------------------------------------------------------------------
// The same computation for callers that cannot allocate: see attention_decode_noalloc.h.
#include <atomic>

#include "attention_decode_noalloc.h"

namespace vob {
// Partial results of the split-key kernel, inside the library.  In host code this name is only a
// stand-in for the symbol, never a device address: the address is looked up below.
static __device__ __align__(256) float g_decode_noalloc_scratch[VOB_DECODE_NOALLOC_MAX_FLOATS];
constexpr int NOALLOC_MAX_DEVICES = 64;
// The array's address per device.  Two host threads may both find an entry empty and both look the address up: they
// store the same value, so the race is harmless; the atomic only keeps the read and the write whole.
static std::atomic<float*> g_decode_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};
}  // namespace vob

VOB_API long vob_attention_decode_noalloc_max_floats(void) { return VOB_DECODE_NOALLOC_MAX_FLOATS; }

VOB_API const char* vob_attention_decode_noalloc_error(int code) {
  if (code == VOB_NOALLOC_TOO_LARGE)
    return "vob_attention_decode_noalloc: num_requests * nh * num_splits * (head size + 1) floats exceed the built-in "
           "scratch array (VOB_DECODE_NOALLOC_MAX_FLOATS); use fewer splits or vob_attention_decode with your own scratch";
  if (code == VOB_NOALLOC_NO_DEVICE) return "vob_attention_decode_noalloc: the current device index is out of range";
  if (code == VOB_BAD_ARGUMENT) return "vob_attention_decode_noalloc: bad argument";
  if (code == VOB_UNSUPPORTED) return "vob_attention_decode_noalloc: size not supported by the decode kernel";
  return cudaGetErrorString((cudaError_t)code);
}

VOB_API int vob_attention_decode_noalloc(const void* q, long q_stride, void* out, const void* kcache, const void* vcache,
                                         const int* block_tables, int table_stride, const int* cu_q,
                                         const int* context_lens, int num_requests, int nh, int kvh, int block_size,
                                         int window, float scale, long num_pages, int num_splits, int* err,
                                         cudaStream_t stream) {
  if (num_requests <= 0) return 0;
  // every argument is looked at before the device is: a call that is refused has touched nothing
  if (num_splits < 1 || nh <= 0 || kvh <= 0 || nh % kvh || block_size <= 0 || !q || !out || !kcache || !vcache ||
      !block_tables || !cu_q || !context_lens || !err)
    return VOB_BAD_ARGUMENT;
  const long need = vob_attention_decode_scratch_floats(num_requests, nh, num_splits);
  if (need > VOB_DECODE_NOALLOC_MAX_FLOATS) return VOB_NOALLOC_TOO_LARGE;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return VOB_NOALLOC_NO_DEVICE;
  float* ptr = g_decode_noalloc_ptr[dev].load(std::memory_order_acquire);
  if (!ptr) {   // set-up, once per device, with that device current
    e = cudaGetSymbolAddress((void**)&ptr, g_decode_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    g_decode_noalloc_ptr[dev].store(ptr, std::memory_order_release);
  }
  return vob_attention_decode(q, q_stride, out, kcache, vcache, block_tables, table_stride, cu_q, context_lens,
                              num_requests, nh, kvh, block_size, window, scale, num_pages, num_splits, ptr, err, stream);
}
