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
#define VOB_TIMEOUT_WHERE 0x800
#include "attention_mma.cuh"

namespace vob {

constexpr int PF_TILE = 64;
constexpr int PF_WARPS = 4;
constexpr int PF_ROWS = PF_WARPS * 16;
constexpr int PF_STAGES = HD <= 128 ? 3 : 2;
constexpr int PF_STAGE_BYTES = 2 * PF_TILE * ROW_BYTES;

__global__ void __launch_bounds__(PF_WARPS * 32)
attention_prefill_kernel(const __nv_bfloat16* q, long q_stride, __nv_bfloat16* out,
                         const __nv_bfloat16* kcache, const __nv_bfloat16* vcache,
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
  const int row0 = (int)(gridDim.x - 1 - blockIdx.x) * PF_ROWS;   // longest blocks first
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

#if VOB_HD % 64 == 0
// ---- the same attention with TMA copies, 128 rows per block and 64 keys per softmax step ----------------
// For head sizes that are a multiple of 64 (head sizes 64 and 128 normally take the tcgen05 kernel of
// attention_prefill_tc5.cu instead).  Eight consumer warps own 16 rows each (128 rows: twice the reuse of every key
// and value brought in); a ninth warp is the producer: its lanes look the pages of eight tiles up at once, a chunk
// ahead, and one thread issues one TMA copy of K and one of V per tile (per run of 16 keys when pages do not hold
// a multiple of 64), into a ring of stages guarded by mbarriers with bounded waits.  A consumer multiplies
// its rows with all 64 keys of a tile before it updates the running maximum, so the accumulator is rescaled
// once per tile; tiles that need no mask (wholly below the diagonal and inside the window) skip the masking.
constexpr int PT_WARPS = 8;
constexpr int PT_ROWS = PT_WARPS * 16;
constexpr int PT_TILE = 64;
constexpr int PT_SLICES = HD / 64;
constexpr int PT_TILE_BYTES = PT_SLICES * PT_TILE * 128;     // one of K or V
constexpr int PT_STAGE_BYTES = 2 * PT_TILE_BYTES;
constexpr int PT_STAGES = HD <= 128 ? 4 : 2;
constexpr int PT_THREADS = (PT_WARPS + 1) * 32;

__global__ void __launch_bounds__(PT_THREADS, 1)
attention_prefill_tma_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                             const __nv_bfloat16* q, long q_stride, __nv_bfloat16* out,
                             const int* __restrict__ block_tables, int table_stride, const int* __restrict__ cu_q,
                             const int* __restrict__ context_lens, int nh, int kvh, int block_size, int window, float scale,
                             long num_pages, int box_keys, int* err) {
  extern __shared__ __align__(1024) char smem_raw[];
  char* smem = reinterpret_cast<char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + PT_STAGES * PT_STAGE_BYTES);
  uint64_t* empty = full + PT_STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + PT_STAGES);
  pdl_launch_dependents();
  const int kh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < PT_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], PT_WARPS); }
    *abort_flag = 0;
    tma_prefetch_map(&tmK);
    tma_prefetch_map(&tmV);
  }
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  __syncthreads();
  pdl_wait();
  const int t0 = cu_q[b];
  const int n = cu_q[b + 1] - t0;
  if (n <= 1) return;                                   // nothing, or a decoding request
  const int G = nh / kvh;
  const int total_rows = n * G;
  // later row blocks see more keys: they go first, so that the short ones fill the end of the grid
  const int row0 = (int)(gridDim.x - 1 - blockIdx.x) * PT_ROWS;
  if (row0 >= total_rows) return;
  const int ctx = context_lens[b];
  const int first_pos = ctx - n;
  const int* table = block_tables + (size_t)b * table_stride;
  const int last_row = min(row0 + PT_ROWS, total_rows) - 1;
  const int blk_pos_lo = first_pos + row0 / G, blk_pos_hi = first_pos + last_row / G;
  const int key_lo = window > 0 ? max(0, blk_pos_lo - window + 1) : 0;
  const int key_end = blk_pos_hi + 1;
  const int start = key_lo / PT_TILE * PT_TILE;
  const int n_tiles = (key_end - start + PT_TILE - 1) / PT_TILE;

  if (warp == PT_WARPS) {
    // ------------------------------------------------ producer: lane 0 issues, all lanes look pages up
    {
      WarpPages wp;
      bool ok = true;
      int it = 0;
      for (; it < n_tiles; ++it) {
        const int s = it % PT_STAGES;
        wp.advance(table, block_size, start, it, lane, key_lo, key_end);
        int pg[4];
#pragma unroll
        for (int run = 0; run < 4; ++run) pg[run] = wp.page(it, run);
        if (lane == 0) {
          if (it >= PT_STAGES) ok = mbar_wait(&empty[s], (unsigned)(((it / PT_STAGES) - 1) & 1), abort_flag, err);
          if (ok) {
            const int tile_start = start + it * PT_TILE;
            mbar_expect_tx(&full[s], (unsigned)PT_STAGE_BYTES);
            char* kt = smem + s * PT_STAGE_BYTES;
            if (box_keys == PT_TILE) {
              // the tile lies in one page: one copy of K, one of V (any run that is wanted names the page)
              const int page = pg[0] != PAGE_NONE ? pg[0] : (pg[1] != PAGE_NONE ? pg[1] : (pg[2] != PAGE_NONE ? pg[2] : pg[3]));
              const bool page_ok = page >= 0 && page < num_pages;
              if (!page_ok && page != PAGE_NONE) atomicOr(err, VOB_ERR_PAGE);
              const int row = page_ok ? (page * kvh + kh) * block_size + tile_start % block_size : 0;
              tma_load_3d(kt, &tmK, 0, row, 0, &full[s]);
              tma_load_3d(kt + PT_TILE_BYTES, &tmV, 0, row, 0, &full[s]);
            } else {
#pragma unroll
              for (int run = 0; run < 4; ++run) {
                const bool page_ok = pg[run] >= 0 && pg[run] < num_pages;
                if (!page_ok && pg[run] != PAGE_NONE) atomicOr(err, VOB_ERR_PAGE);
                // a run nobody will read is filled from row 0 of the plane: finite values that the mask zeroes
                const int key0 = tile_start + run * RUN_KEYS;
                const int row = page_ok ? (pg[run] * kvh + kh) * block_size + key0 % block_size : 0;
                // a 16-row box writes its slices 16 rows apart, the tile keeps them PT_TILE rows apart: a copy per slice
#pragma unroll
                for (int c = 0; c < PT_SLICES; ++c) {
                  tma_load_3d(kt + c * PT_TILE * 128 + run * RUN_KEYS * 128, &tmK, 0, row, c, &full[s]);
                  tma_load_3d(kt + PT_TILE_BYTES + c * PT_TILE * 128 + run * RUN_KEYS * 128, &tmV, 0, row, c, &full[s]);
                }
              }
            }
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
      }
      if (lane == 0) {
        const int first = it > PT_STAGES ? it - PT_STAGES : 0;     // copies in flight must land before the block exits
        for (int j = first; j < it; ++j) {
          bool done = false;
          for (unsigned i = 0; i < MBAR_SPIN_LIMIT && !done; ++i) done = mbar_try_wait(&full[j % PT_STAGES], (unsigned)((j / PT_STAGES) & 1));
          if (!done) atomicOr(err, VOB_ERR_TIMEOUT_BITS);
        }
      }
    }
    return;
  }
  // ------------------------------------------------ consumers: 16 rows per warp
  const int g = lane >> 2, tq = lane & 3;
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
  const int w_first = min(row0 + warp * 16, last_row), w_last = min(row0 + warp * 16 + 15, last_row);
  const int w_pos_lo = first_pos + w_first / G, w_pos_hi = first_pos + w_last / G;
  const int w_key_lo = window > 0 ? max(0, w_pos_lo - window + 1) : 0;
  const bool warp_active = row0 + warp * 16 < total_rows;
  const bool all_rows = row0 + warp * 16 + 15 < total_rows;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[DTILES][4];
#pragma unroll
  for (int j = 0; j < DTILES; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  const float sc = scale * LOG2E;
  const int mi = lane >> 3, r8 = lane & 7;

  for (int it = 0; it < n_tiles; ++it) {
    const int s = it % PT_STAGES;
    bool ok = mbar_wait(&full[s], (unsigned)((it / PT_STAGES) & 1), abort_flag, err);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    const char* kt = smem + s * PT_STAGE_BYTES;
    const char* vt = kt + PT_TILE_BYTES;
    const int k0 = start + it * PT_TILE;
    if (warp_active && k0 <= w_pos_hi && k0 + PT_TILE > w_key_lo) {
      // scores of 16 rows against 64 keys
      float sv[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) sv[i][0] = sv[i][1] = sv[i][2] = sv[i][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        const char* slice = kt + (ks >> 2) * PT_TILE * 128;
        const int chunk = (ks & 3) * 2 + (mi & 1);
#pragma unroll
        for (int kg = 0; kg < 4; ++kg) {
          uint32_t bk[4];
          ldmatrix_x4(bk, slice + swizzled_offset(kg * 16 + (mi >> 1) * 8 + r8, chunk));
          mma_bf16(sv[2 * kg], qf[ks], bk[0], bk[1]);
          mma_bf16(sv[2 * kg + 1], qf[ks], bk[2], bk[3]);
        }
      }
      // mask only where the tile touches the diagonal, the window's edge, the range's ends or missing rows
      const bool need_mask = !all_rows || k0 + PT_TILE - 1 > w_pos_lo || k0 < key_lo ||
                             (window > 0 && k0 < w_pos_hi - window + 1);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int h = e >> 1;
            const int key = k0 + i * 8 + tq * 2 + (e & 1);
            bool okk = rvalid[h] && key <= rpos[h] && key >= key_lo;
            if (window > 0) okk = okk && key > rpos[h] - window;
            sv[i][e] = okk ? sv[i][e] * sc : -INFINITY;
          }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) { sv[i][0] *= sc; sv[i][1] *= sc; sv[i][2] *= sc; sv[i][3] *= sc; }
      }
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        mx[0] = fmaxf(mx[0], fmaxf(sv[i][0], sv[i][1]));
        mx[1] = fmaxf(mx[1], fmaxf(sv[i][2], sv[i][3]));
      }
      float corr[2], mu[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float mnew = fmaxf(m[h], mx[h]);
        corr[h] = (m[h] == -INFINITY) ? 0.f : fast_exp2(m[h] - mnew);
        m[h] = mnew;
        mu[h] = mnew == -INFINITY ? 0.f : mnew;
      }
      float sum[2] = {0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        sv[i][0] = fast_exp2(sv[i][0] - mu[0]); sv[i][1] = fast_exp2(sv[i][1] - mu[0]);
        sv[i][2] = fast_exp2(sv[i][2] - mu[1]); sv[i][3] = fast_exp2(sv[i][3] - mu[1]);
        sum[0] += sv[i][0] + sv[i][1];
        sum[1] += sv[i][2] + sv[i][3];
      }
      l[0] = l[0] * corr[0] + sum[0];
      l[1] = l[1] * corr[1] + sum[1];
#pragma unroll
      for (int j = 0; j < DTILES; ++j) { o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1]; }
      // o += P * V, 16 keys at a time
#pragma unroll
      for (int kg = 0; kg < 4; ++kg) {
        uint32_t a[4];
        a[0] = pack_bf16(sv[2 * kg][0], sv[2 * kg][1]);
        a[1] = pack_bf16(sv[2 * kg][2], sv[2 * kg][3]);
        a[2] = pack_bf16(sv[2 * kg + 1][0], sv[2 * kg + 1][1]);
        a[3] = pack_bf16(sv[2 * kg + 1][2], sv[2 * kg + 1][3]);
        const int vrow = kg * 16 + (mi & 1) * 8 + r8;
#pragma unroll
        for (int j = 0; j < DTILES; j += 2) {
          const int d0 = j * 8 + (mi >> 1) * 8;
          uint32_t bv[4];
          ldmatrix_x4_trans(bv, vt + (d0 >> 6) * PT_TILE * 128 + swizzled_offset(vrow, (d0 & 63) >> 3));
          mma_bf16(o[j], a, bv[0], bv[1]);
          mma_bf16(o[j + 1], a, bv[2], bv[3]);
        }
      }
    }
    // ordinary loads of the stage before the copy engine's next write to it: a proxy fence, then the release
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
  }
  if (*abort_flag) return;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (!rvalid[h]) continue;
    const float inv = l[h] > 0.f ? 1.f / l[h] : 0.f;
    __nv_bfloat16* orow = out + (size_t)(t0 + rtok[h]) * nh * HD + (size_t)rhead[h] * HD + tq * 2;
#pragma unroll
    for (int j = 0; j < DTILES; ++j)
      *reinterpret_cast<__nv_bfloat162*>(orow + j * 8) = __floats2bfloat162_rn(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
  }
}
#endif  // VOB_HD % 64 == 0

}  // namespace vob

using namespace vob;

static int attention_prefill_launch(const void* map_k, const void* map_v, const void* q, long q_stride, void* out,
                                    const void* kcache, const void* vcache, const int* block_tables, int table_stride,
                                    const int* cu_q, const int* context_lens, int num_requests, int max_q, int nh, int kvh,
                                    int block_size, int window, float scale, long num_pages, int* err, cudaStream_t stream) {
  if (num_requests <= 0 || max_q <= 1) return 0;
  if (kvh <= 0 || nh % kvh || block_size <= 0 || kvh > 65535 || num_requests > 65535) return VOB_UNSUPPORTED;
  const long rows = (long)max_q * (nh / kvh);
#if VOB_HD % 64 == 0
  if (map_k && map_v && block_size % 16 == 0) {
    static bool tma_configured = false;
    const int tma_smem = 1024 + PT_STAGES * PT_STAGE_BYTES + 2 * PT_STAGES * 8 + 16;
    if (!tma_configured) {
      cudaError_t e = cudaFuncSetAttribute(attention_prefill_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, tma_smem);
      if (e != cudaSuccess) return (int)e;
      tma_configured = true;
    }
    dim3 grid((unsigned)((rows + PT_ROWS - 1) / PT_ROWS), kvh, num_requests);
    return launch_kernel(attention_prefill_tma_kernel, grid, PT_THREADS, tma_smem, stream, *(const CUtensorMap*)map_k,
                         *(const CUtensorMap*)map_v, (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, block_tables,
                         table_stride, cu_q, context_lens, nh, kvh, block_size, window, scale, num_pages,
                         block_size % PT_TILE == 0 ? PT_TILE : RUN_KEYS, err);
  }
#endif
  static bool configured = false;
  const int smem = PF_STAGES * PF_STAGE_BYTES;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((unsigned)((rows + PF_ROWS - 1) / PF_ROWS), kvh, num_requests);
  return launch_kernel(attention_prefill_kernel, grid, PF_WARPS * 32, smem, stream, (const __nv_bfloat16*)q, q_stride,
                       (__nv_bfloat16*)out, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, block_tables,
                       table_stride, cu_q, context_lens, nh, kvh, block_size, window, scale, num_pages, err);
}

// max_q: the most tokens any request brings in this step (sizes the grid).
VOB_API int vob_attention_prefill(const void* q, long q_stride, void* out, const void* kcache, const void* vcache,
                                  const int* block_tables, int table_stride, const int* cu_q, const int* context_lens,
                                  int num_requests, int max_q, int nh, int kvh, int block_size, int window, float scale,
                                  long num_pages, int* err, cudaStream_t stream) {
  return attention_prefill_launch(nullptr, nullptr, q, q_stride, out, kcache, vcache, block_tables, table_stride, cu_q,
                                  context_lens, num_requests, max_q, nh, kvh, block_size, window, scale, num_pages, err, stream);
}

// The same with the caches also given as tensor maps (as for vob_attention_decode_tma): head sizes that are a
// multiple of 64 then take the TMA kernel.
VOB_API int vob_attention_prefill_tma(const void* map_k, const void* map_v, const void* q, long q_stride, void* out,
                                      const void* kcache, const void* vcache, const int* block_tables, int table_stride,
                                      const int* cu_q, const int* context_lens, int num_requests, int max_q, int nh,
                                      int kvh, int block_size, int window, float scale, long num_pages, int* err,
                                      cudaStream_t stream) {
  return attention_prefill_launch(map_k, map_v, q, q_stride, out, kcache, vcache, block_tables, table_stride, cu_q,
                                  context_lens, num_requests, max_q, nh, kvh, block_size, window, scale, num_pages, err, stream);
}
