// Causal attention of prompt portions over the paged cache on the fifth-generation tensor cores, for head sizes
// 64 and 128: S = Q K^T and O = P V are tcgen05.mma products with S and O in tensor memory.
//
// A block takes NQ tiles of 128 query rows (a row is a (token, head of the group) pair, so the heads that share a
// key/value head share every key and value brought in; a tile holds whole tokens, 128 / group of them, and leaves the
// rows that remain, two of 128 with three heads a group, as zeros) and walks the keys in steps of 64:
//   warps 0 .. 4NQ-1   softmax: warp w of a tile owns rows 32(w%4) .. +31 of it, a thread owns ONE row: it reads the
//                      row's 64 scores from tensor memory (tcgen05.ld), masks, takes the maximum and the sum without
//                      any exchange between threads, writes P in bfloat16 back to tensor memory over the scores (the A
//                      operand of the second product), and at the end divides the row of O by its sum and stores it:
//                      a whole tile through shared memory (where the query tile lay) and one TMA store a 64-column
//                      slice, a tile with rows past the request's end row by row (32 bytes a store).  From a row's
//                      second step on the exponentials are taken against the old reference maximum beside the search
//                      for the new one, and taken again only if it had to move;
//   warp 4NQ           producer: brings the query tiles in (TMA: the tensor map sees q as head size x heads x tokens, a
//                      box is 64 columns of a group's heads for a tile's tokens and lands as the tile's rows; for a
//                      caller without that map the softmax warps bring them by cp.async instead),
//                      looks the pages up a chunk ahead and brings K and V tiles in by TMA into a ring of
//                      stages (the K tile is the K-major B operand of the first product as it lands, the V tile the
//                      MN-major B operand of the second one: no transposition anywhere);
//   warps 4NQ+1 ..     one per query tile (the first of them allocates tensor memory): a thread issues the tile's
//                      products, the scores of step j+1 into a second S buffer while the softmax of step j runs;
//                      tcgen05.commit tells the softmax warps that S is complete and that O has been updated, and
//                      the producer that the tile is done with a stage.  The tiles do not wait for one another.
// At a block's start the producer asks for its first pages before the barriers are set up and goes for the query
// tiles and the first keys and values as soon as they exist, while tensor memory is allocated.
// A wait on an mbarrier goes by the parity of the phase, so it can tell only two states apart: the scores and P have
// a barrier per buffer (a buffer's next use needs the waiter's own progress).  O's barrier gets a phase per step; a
// softmax thread that has to rescale O at step i waits on it for step i - 1, when it can be in two states only (that
// product pending or done: the next one needs this thread's own P).  At the end it could be in three (the last two
// products pending, the last one, none), so the end of a tile's last product has a barrier of its own, used once.
// O stays in tensor memory over all steps.  The running maximum that the exponentials refer to is moved only when a
// row's new maximum exceeds it by more than 8 (in base-2 units: P stays below 256, exact enough in bfloat16 since
// its error is relative); only then the row's O is read, scaled and written back, which is rare after the first
// steps.  Sums, maxima and the scaling are in float.  Every wait on an mbarrier is bounded; a block that gives up
// sets an error bit, stops issuing work, waits for what is in flight, and frees its tensor memory.
#define VOB_TIMEOUT_WHERE 0x1000
#include "attention_mma.cuh"
#include "tcgen05.cuh"

namespace vob {

#if VOB_HD == 64 || VOB_HD == 128

constexpr int F5_ROWS = 128;                               // rows of a query tile (the MMA's M)
constexpr int F5_TILE = 64;                                // keys per step
constexpr int F5_SLICES = HD / 64;                         // 64-column slices of a head
constexpr int F5_Q_BYTES = F5_SLICES * F5_ROWS * 128;      // a query tile: [slice][128 rows][128 bytes]
constexpr int F5_KV_BYTES = F5_SLICES * F5_TILE * 128;     // one of K or V: [slice][64 keys][128 bytes]
constexpr int F5_STAGE_BYTES = 2 * F5_KV_BYTES;
constexpr float F5_MAX_SLACK = 8.f;                        // how far a row's maximum may run ahead of its reference

template <int NQ> struct F5 {
  static constexpr int THREADS = (5 * NQ + 1) * 32;        // 4 softmax warps and one issuing warp per tile, a producer
  // One tile a block: two blocks share an SM (half the shared memory and half the tensor memory each).  Two tiles a
  // block: one block per SM.  Shared memory left after the query tiles goes to the ring of K/V stages.
  static constexpr int BLOCKS_PER_SM = NQ == 1 ? 2 : 1;
  static constexpr int STAGES = (220 * 1024 / BLOCKS_PER_SM - NQ * F5_Q_BYTES) / F5_STAGE_BYTES;
  static constexpr int TILE_COLS = 2 * F5_TILE + HD;       // tensor-memory columns of a query tile: S, S, O
  static constexpr int TMEM_COLS = NQ * TILE_COLS <= 256 ? 256 : 512;
  static constexpr int DATA_BYTES = NQ * F5_Q_BYTES + STAGES * F5_STAGE_BYTES;
  static constexpr int NUM_BARRIERS = 2 * STAGES + 8 * NQ + 1;
  static constexpr int SMEM_BYTES = 1024 + DATA_BYTES + NUM_BARRIERS * 8 + 16;
};

template <int NQ>
__global__ void __launch_bounds__(F5<NQ>::THREADS, F5<NQ>::BLOCKS_PER_SM)
attention_prefill_tc5_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                             const __grid_constant__ CUtensorMap tmQ, int q_by_tma,
                             const __grid_constant__ CUtensorMap tmO, int o_by_tma,
                             const __nv_bfloat16* q, long q_stride, __nv_bfloat16* out,
                             const int* __restrict__ block_tables, int table_stride, const int* __restrict__ cu_q,
                             const int* __restrict__ context_lens, int nh, int kvh, int block_size, int window, float scale,
                             long num_pages, int box_keys, int* err) {
  using C = F5<NQ>;
  constexpr int ST = C::STAGES;
  extern __shared__ __align__(1024) char smem_raw[];
  char* smem = reinterpret_cast<char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  char* q_s = smem;                                         // [NQ] query tiles
  char* kv_s = q_s + NQ * F5_Q_BYTES;                       // [ST] stages: K tile, V tile
  uint64_t* kv_full = reinterpret_cast<uint64_t*>(smem + C::DATA_BYTES);
  uint64_t* kv_empty = kv_full + ST;
  uint64_t* s_full = kv_empty + ST;                         // [NQ][2] scores of a step are complete
  uint64_t* p_full = s_full + 2 * NQ;                       // [NQ][2] P of a step is written (and S read, O rescaled)
  uint64_t* o_done = p_full + 2 * NQ;                       // [NQ] O holds the step's contribution
  uint64_t* o_final = o_done + NQ;                          // [NQ] O holds the last step's contribution (one phase)
  uint64_t* drained = o_final + NQ;                         // every product issued has completed
  uint64_t* q_full = drained + 1;                           // [NQ] the query tile has landed (when TMA brings it)
  uint64_t* o_staged = q_full + NQ;                         // [NQ] the tile's four warps have put their rows of O in shared memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_staged + NQ);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  pdl_launch_dependents();
  // blockIdx.x = row block * kv heads + kv head: the blocks of all heads that see the most keys start first
  const int kh = blockIdx.x % kvh, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = cu_q[b];
  const int n = cu_q[b + 1] - t0;
  const int G = nh / kvh;
  // A tile holds whole tokens: TT of them, TR = TT * G rows (126 of the 128 with three heads a group; the rows that are
  // left are zeros that nobody reads).  So a tile never ends inside a token, and one box of a tensor map is a tile.
  const int TT = F5_ROWS / G, TR = TT * G;
  // later blocks of tokens see more keys: they go first, so that the short ones fill the end of the grid
  const int tok_base = (int)(gridDim.x / kvh - 1 - blockIdx.x / kvh) * NQ * TT;
  if (n <= 1 || tok_base >= n) { pdl_wait(); return; }             // a decoding request, or nothing left (uniform)
  const int ctx = context_lens[b];
  const int first_pos = ctx - n;
  const int* table = block_tables + (size_t)b * table_stride;
  const int blk_pos_lo = first_pos + tok_base, blk_pos_hi = first_pos + min(tok_base + NQ * TT, n) - 1;
  const int key_lo = window > 0 ? max(0, blk_pos_lo - window + 1) : 0;
  const int key_end = blk_pos_hi + 1;
  const int start = key_lo / F5_TILE * F5_TILE;
  const int n_tiles = (key_end - start + F5_TILE - 1) / F5_TILE;
  // the steps that each query tile takes part in: [jlo, jhi)
  int jlo[NQ], jhi[NQ];
#pragma unroll
  for (int qt = 0; qt < NQ; ++qt) {
    const int tok_first = tok_base + qt * TT;
    if (tok_first >= n) { jlo[qt] = jhi[qt] = 0; continue; }
    const int pos_lo = first_pos + tok_first, pos_hi = first_pos + min(tok_first + TT, n) - 1;
    const int klo = window > 0 ? max(0, pos_lo - window + 1) : 0;
    jlo[qt] = (klo - start) / F5_TILE;
    jhi[qt] = (pos_hi - start) / F5_TILE + 1;
  }

  // the producer asks for the pages of its first tiles now (the block tables were written before the step began), so
  // that the look-up runs beside the set-up below
  WarpPages wp;
  if (warp == 4 * NQ) wp.advance(table, block_size, start, 0, lane, key_lo, key_end);
  if (threadIdx.x == 0) {
    for (int s = 0; s < ST; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], NQ); }
    for (int i = 0; i < 2 * NQ; ++i) { mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 4); }
    for (int i = 0; i < NQ; ++i) {
      mbar_init(&o_done[i], 1); mbar_init(&o_final[i], 1); mbar_init(&q_full[i], 1); mbar_init(&o_staged[i], 4);
    }
    mbar_init(drained, NQ);
    *abort_flag = 0;
    tma_prefetch_map(&tmK);
    tma_prefetch_map(&tmV);
    if (q_by_tma) tma_prefetch_map(&tmQ);
    if (o_by_tma) tma_prefetch_map(&tmO);
  }
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  __syncthreads();                              // the barriers are there: the producer starts on the first keys and values
  pdl_wait();                                   // the kernels before this one wrote q and this portion's keys and values
  uint32_t tmem_base = 0;
  if (warp != 4 * NQ) {
    if (warp == 4 * NQ + 1) t5_alloc(tmem_slot, C::TMEM_COLS);
    if (warp < 4 * NQ && TR < F5_ROWS) {
      // the rows of a tile that hold no token: zeros (finite scores that nobody reads)
      const int qt = warp >> 2, tid = threadIdx.x & 127;
      for (int idx = tid; idx < F5_SLICES * (F5_ROWS - TR) * 8; idx += 128) {
        const int c = idx / ((F5_ROWS - TR) * 8), rest = idx % ((F5_ROWS - TR) * 8);
        *reinterpret_cast<uint4*>(q_s + qt * F5_Q_BYTES + c * (F5_ROWS * 128) + (TR + rest / 8) * 128 + (rest % 8) * 16) =
            make_uint4(0u, 0u, 0u, 0u);
      }
    }
    if (warp < 4 * NQ && !q_by_tma) {
      // the query tile of this warp group into shared memory, rows of 128 bytes per slice, 128-byte swizzled; every
      // copy is on its way before the first one is waited for (cp.async moves 16 bytes a clock: 4,000 cycles for two
      // tiles, which is why the copy engine brings them where it can)
      const int qt = warp >> 2, tid = threadIdx.x & 127;
      char* dst = q_s + qt * F5_Q_BYTES;
      constexpr int CHUNKS = HD / 8;
#pragma unroll 4
      for (int idx = tid; idx < TR * CHUNKS; idx += 128) {
        const int r = idx / CHUNKS, chunk = idx % CHUNKS;
        const int tok = tok_base + qt * TT + r / G;
        const bool there = tok < n;
        const __nv_bfloat16* src = there ? q + (size_t)(t0 + tok) * q_stride + (size_t)(kh * G + r % G) * HD + chunk * 8 : q;
        cp_async16(dst + (chunk >> 3) * (F5_ROWS * 128) + swizzled_offset(r, chunk & 7), src, there);
      }
      cp_async_commit();
      cp_async_wait<0>();
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    t5_fence_before();
    asm volatile("bar.sync 1, %0;\n" ::"n"(5 * NQ * 32) : "memory");   // the softmax and the issuing warps
    t5_fence_after();
    tmem_base = *tmem_slot;
  }

  if (warp == 4 * NQ) {
    // ------------------------------------------------ producer: lane 0 issues, all lanes look pages up
    if (q_by_tma && lane == 0) {
      // The query tiles by the copy engine: the tensor map sees q as (head size, heads, tokens), a box is 64 columns of
      // the G heads of a kv head for TT tokens, which lands as TR rows of 128 bytes in the order (token, head of the
      // group): the tile's rows.  Tokens past the step's last read as zeros; rows past the request's are masked.
#pragma unroll
      for (int qt = 0; qt < NQ; ++qt) {
        if (jhi[qt] > jlo[qt]) {
          mbar_expect_tx(&q_full[qt], (unsigned)(F5_SLICES * TR * 128));
#pragma unroll
          for (int c = 0; c < F5_SLICES; ++c)
            tma_load_3d(q_s + qt * F5_Q_BYTES + c * (F5_ROWS * 128), &tmQ, c * 64, kh * G, t0 + tok_base + qt * TT, &q_full[qt]);
        }
      }
    }
    bool ok = true;
    int it = 0;
    for (; it < n_tiles; ++it) {
      const int s = it % ST;
      if (it > 0) wp.advance(table, block_size, start, it, lane, key_lo, key_end);
      int pg[4];
#pragma unroll
      for (int run = 0; run < 4; ++run) pg[run] = wp.page(it, run);
      if (lane == 0) {
        if (it >= ST) ok = mbar_wait(&kv_empty[s], (unsigned)(((it / ST) - 1) & 1), abort_flag, err);
        if (ok) {
          const int tile_start = start + it * F5_TILE;
          mbar_expect_tx(&kv_full[s], (unsigned)F5_STAGE_BYTES);
          char* kt = kv_s + s * F5_STAGE_BYTES;
          if (box_keys == F5_TILE) {
            // the tile lies in one page: one copy of K, one of V (any run that is wanted names the page)
            const int page = pg[0] != PAGE_NONE ? pg[0] : (pg[1] != PAGE_NONE ? pg[1] : (pg[2] != PAGE_NONE ? pg[2] : pg[3]));
            const bool page_ok = page >= 0 && page < num_pages;
            if (!page_ok && page != PAGE_NONE) atomicOr(err, VOB_ERR_PAGE);
            const int row = page_ok ? (page * kvh + kh) * block_size + tile_start % block_size : 0;
            tma_load_3d(kt, &tmK, 0, row, 0, &kv_full[s]);
            tma_load_3d(kt + F5_KV_BYTES, &tmV, 0, row, 0, &kv_full[s]);
          } else {
#pragma unroll
            for (int run = 0; run < 4; ++run) {
              const bool page_ok = pg[run] >= 0 && pg[run] < num_pages;
              if (!page_ok && pg[run] != PAGE_NONE) atomicOr(err, VOB_ERR_PAGE);
              // a run nobody will read is filled from row 0 of the plane: finite values that the mask zeroes
              const int key0 = tile_start + run * RUN_KEYS;
              const int row = page_ok ? (pg[run] * kvh + kh) * block_size + key0 % block_size : 0;
#pragma unroll
              for (int c = 0; c < F5_SLICES; ++c) {
                tma_load_3d(kt + c * F5_TILE * 128 + run * RUN_KEYS * 128, &tmK, 0, row, c, &kv_full[s]);
                tma_load_3d(kt + F5_KV_BYTES + c * F5_TILE * 128 + run * RUN_KEYS * 128, &tmV, 0, row, c, &kv_full[s]);
              }
            }
          }
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
    }
    if (lane == 0) {
      if (q_by_tma) {                              // (the query tiles too, should their tile have given up before it saw them)
#pragma unroll
        for (int qt = 0; qt < NQ; ++qt) {
          bool done = jhi[qt] <= jlo[qt];
          for (unsigned i = 0; i < MBAR_SPIN_LIMIT && !done; ++i) done = mbar_try_wait(&q_full[qt], 0u);
          if (!done) atomicOr(err, VOB_ERR_TIMEOUT_BITS);
        }
      }
      const int first = it > ST ? it - ST : 0;     // copies in flight must land before the block exits
      for (int j = first; j < it; ++j) {
        bool done = false;
        for (unsigned i = 0; i < MBAR_SPIN_LIMIT && !done; ++i) done = mbar_try_wait(&kv_full[j % ST], (unsigned)((j / ST) & 1));
        if (!done) atomicOr(err, VOB_ERR_TIMEOUT_BITS);
      }
    }
  } else if (warp > 4 * NQ) {
    // ------------------------------------------------ the products of query tile qt (one thread per tile)
    if (lane == 0) {
      const int qt = warp - (4 * NQ + 1);
      const uint32_t idesc_qk = t5_instr_desc(F5_ROWS, F5_TILE);
      const uint32_t idesc_pv = t5_instr_desc_b_mn(F5_ROWS, HD);
      const int lo = jlo[qt], hi = jhi[qt];
      const uint32_t s_tmem = tmem_base + qt * C::TILE_COLS, o_tmem = s_tmem + 2 * F5_TILE;
      // descriptors differ from one k-step or stage to the next only in the start address (in units of 16 bytes)
      const uint64_t q_desc = t5_smem_desc(q_s + qt * F5_Q_BYTES);
      const uint64_t k_desc0 = t5_smem_desc(kv_s);
      const uint64_t v_desc0 = t5_smem_desc_mn(kv_s + F5_KV_BYTES, F5_TILE * 128, 1024);
      bool ok = true;
      if (q_by_tma && hi > lo) ok = mbar_wait(&q_full[qt], 0u, abort_flag, err);
      // S[buffer] = Q K_j^T
      auto scores = [&](int j) {
        const int i = j - lo;
        const uint64_t kd = k_desc0 + (uint64_t)(((j % ST) * F5_STAGE_BYTES) >> 4);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          t5_mma(s_tmem + (i & 1) * F5_TILE, q_desc + (uint64_t)(((ks >> 2) * (F5_ROWS * 128) + (ks & 3) * 32) >> 4),
                 kd + (uint64_t)(((ks >> 2) * (F5_TILE * 128) + (ks & 3) * 32) >> 4), idesc_qk, ks > 0);
        t5_commit(&s_full[qt * 2 + (i & 1)]);
      };
      for (int j = 0; ok && j < n_tiles; ++j) {
        if (j < lo || j >= hi) {
          // this tile does not need the step's keys: it only tells the producer so, once they have arrived
          ok = mbar_wait(&kv_full[j % ST], (unsigned)((j / ST) & 1), abort_flag, err);
          if (ok) mbar_arrive(&kv_empty[j % ST]);
          continue;
        }
        const int i = j - lo;
        if (i == 0) {
          ok = mbar_wait(&kv_full[j % ST], (unsigned)((j / ST) & 1), abort_flag, err);
          if (!ok) break;
          t5_fence_after();
          scores(j);
        }
        if (j + 1 < hi) {      // the scores of the next step go into the other buffer while this step's softmax runs
          ok = mbar_wait(&kv_full[(j + 1) % ST], (unsigned)(((j + 1) / ST) & 1), abort_flag, err);
          if (!ok) break;
          t5_fence_after();
          scores(j + 1);
        }
        ok = mbar_wait(&p_full[qt * 2 + (i & 1)], (unsigned)((i >> 1) & 1), abort_flag, err);
        if (!ok) break;
        t5_fence_after();
        const uint64_t vd = v_desc0 + (uint64_t)(((j % ST) * F5_STAGE_BYTES) >> 4);
#pragma unroll
        for (int ks = 0; ks < F5_TILE / 16; ++ks)
          t5_mma_a_tmem(o_tmem, s_tmem + (i & 1) * F5_TILE + ks * 8, vd + (uint64_t)((ks * 16 * 128) >> 4), idesc_pv,
                        (i > 0 || ks > 0) ? 1u : 0u);
        t5_commit(&o_done[qt]);
        if (j + 1 == hi) t5_commit(&o_final[qt]);
        t5_commit(&kv_empty[j % ST]);
      }
      // nothing may still read shared or tensor memory when the block ends
      t5_commit(drained);
      bool done = false;
      for (unsigned i = 0; i < MBAR_SPIN_LIMIT && !done; ++i) done = mbar_try_wait(drained, 0u);
      if (!done) atomicOr(err, VOB_ERR_TIMEOUT_BITS);
    }
  } else {
    // ------------------------------------------------ softmax: a thread owns a row
    const int qt = warp >> 2;
    const int r = (warp & 3) * 32 + lane;                   // row of the tile = lane of tensor memory
    const int tok_first = tok_base + qt * TT;                // the tile's first token
    const bool valid = r < TR && tok_first + r / G < n;
    const int tok = valid ? tok_first + r / G : 0, head = kh * G + (valid ? r % G : 0);
    const int rpos = first_pos + tok;
    const int t_pos_lo = first_pos + tok_first, t_pos_hi = first_pos + min(tok_first + TT, n) - 1;
    const bool all_rows = tok_first + TT <= n;               // every token of the tile is the request's
    const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + qt * C::TILE_COLS;
    const float sc = scale * LOG2E;
    float m_ref = -INFINITY, l = 0.f;
    const int my_lo = jlo[qt], my_hi = jhi[qt];
    bool ok = true;
    for (int j = my_lo; j < my_hi; ++j) {
      const int i = j - my_lo;
      ok = mbar_wait(&s_full[qt * 2 + (i & 1)], (unsigned)((i >> 1) & 1), abort_flag, err);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      t5_fence_after();
      const int k0 = start + j * F5_TILE;
      // mask only where the step touches the diagonal, the window's edge or missing rows
      const bool need_mask = !all_rows || k0 + F5_TILE - 1 > t_pos_lo || (window > 0 && k0 < t_pos_hi - window + 1);
      // (the rows past TR of a whole tile hold zeros: their scores are finite and go nowhere)
      float s[64];
      // the row's 64 scores of this step from tensor memory, masked
      auto load_scores = [&]() {
        uint32_t raw[2][32];
        t5_ld32_issue(lane_base + (i & 1) * F5_TILE, raw[0]);
        t5_ld32_issue(lane_base + (i & 1) * F5_TILE + 32, raw[1]);
        t5_wait_ld();
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < 64; ++c) {
            const int key = k0 + c;
            bool okk = valid && key <= rpos;
            if (window > 0) okk = okk && key > rpos - window;
            s[c] = okk ? __uint_as_float(raw[c >> 5][c & 31]) : -INFINITY;
          }
        } else {
#pragma unroll
          for (int c = 0; c < 64; ++c) s[c] = __uint_as_float(raw[c >> 5][c & 31]);
        }
      };
      // the maximum of the raw scores (the scale is positive): four chains of three-input maxima
      auto row_max = [&]() {
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < 64; c += 8) {
#pragma unroll
          for (int h = 0; h < 4; ++h) m4[h] = max3(m4[h], s[c + 2 * h], s[c + 2 * h + 1]);
        }
        return max3(fmaxf(m4[0], m4[1]), m4[2], m4[3]) * sc;
      };
      uint32_t packed[32];
      float sum = 0.f;
      // P = 2^(s * scale - reference) in bfloat16 pairs, and its sum
      auto exponentials = [&](float neg_mu) {
        float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          const float p0 = fast_exp2(fmaf(s[c], sc, neg_mu)), p1 = fast_exp2(fmaf(s[c + 1], sc, neg_mu));
          part[(c >> 1) & 1] += p0;
          part[2 + ((c >> 1) & 1)] += p1;
          packed[c >> 1] = pack_bf16(p0, p1);
        }
        sum = (part[0] + part[1]) + (part[2] + part[3]);
      };
      load_scores();
      // The reference maximum moves only when the row's maximum has run ahead of it, which is rare after a row's
      // first steps.  So from the second step on the exponentials are taken against the old reference at once, beside
      // the search for the maximum (the two do not depend on each other, and the chain of maxima hides behind the
      // exponentials); only if some row of the warp has to move its reference are the scores read again and the
      // step's exponentials taken anew.
      float mx = 0.f;
      bool moved = i == 0;
      if (i > 0) {
        exponentials(m_ref == -INFINITY ? 0.f : -m_ref);
        mx = row_max();
        moved = __any_sync(0xffffffffu, mx > m_ref + F5_MAX_SLACK);
        if (moved) load_scores();
      } else {
        mx = row_max();
      }
      float factor = 1.f;
      if (moved) {
        if (mx > m_ref + F5_MAX_SLACK) {
          factor = m_ref == -INFINITY ? 0.f : fast_exp2(m_ref - mx);
          m_ref = mx;
          l *= factor;
        }
        exponentials(m_ref == -INFINITY ? 0.f : -m_ref);     // a row that has seen no key yet: a finite stand-in
      }
      l += sum;
      // O is touched only to rescale it, and then the product of the step before must have updated it
      const bool rescale = i > 0 && moved;
      if (rescale) {
        ok = mbar_wait(&o_done[qt], (unsigned)((i - 1) & 1), abort_flag, err);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        t5_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t o[32];
          t5_ld32_issue(lane_base + 2 * F5_TILE + c0, o);
          t5_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * factor);
          t5_st32(lane_base + 2 * F5_TILE + c0, o);
        }
        t5_wait_st();
      }
      // P (bfloat16, two keys per 32-bit column) takes the place of the first 32 columns of the scores it was made
      // from: all of them are in registers now, and the buffer's next scores come after the product that reads P
      t5_st32(lane_base + (i & 1) * F5_TILE, packed);
      t5_wait_st();
      t5_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[qt * 2 + (i & 1)]);
    }
    if (ok && my_hi > my_lo) {
      ok = mbar_wait(&o_final[qt], 0u, abort_flag, err);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        t5_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* orow = out + (size_t)(t0 + tok) * nh * HD + (size_t)head * HD;
        if (o_by_tma && all_rows) {
          // A whole tile leaves through shared memory and the copy engine: its rows go, in the layout a load would have
          // written them, where the query tile lay (every product that read it has completed), and one thread sends
          // each 64-column slice with one copy.  A tile with rows past the request's end stores its rows itself.
          char* stage = q_s + qt * F5_Q_BYTES;
#pragma unroll
          for (int c0 = 0; c0 < HD; c0 += 64) {
            uint32_t o[2][32];
            t5_ld32_issue(lane_base + 2 * F5_TILE + c0, o[0]);
            t5_ld32_issue(lane_base + 2 * F5_TILE + c0 + 32, o[1]);
            t5_wait_ld();
#pragma unroll
            for (int c = 0; c < 64; c += 8) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(o[c >> 5][(c & 31)]) * inv, __uint_as_float(o[c >> 5][(c & 31) + 1]) * inv);
              v.y = pack_bf16(__uint_as_float(o[c >> 5][(c & 31) + 2]) * inv, __uint_as_float(o[c >> 5][(c & 31) + 3]) * inv);
              v.z = pack_bf16(__uint_as_float(o[c >> 5][(c & 31) + 4]) * inv, __uint_as_float(o[c >> 5][(c & 31) + 5]) * inv);
              v.w = pack_bf16(__uint_as_float(o[c >> 5][(c & 31) + 6]) * inv, __uint_as_float(o[c >> 5][(c & 31) + 7]) * inv);
              *reinterpret_cast<uint4*>(stage + (c0 >> 6) * (F5_ROWS * 128) + swizzled_offset(r, c >> 3)) = v;
            }
          }
          // the tile's four warps meet on an mbarrier, not on a block barrier: a warp that gave up above never comes,
          // and then the wait runs out (bounded, like every wait here) instead of holding the others for ever
          asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(&o_staged[qt]);
          if ((warp & 3) == 0 && lane == 0 && mbar_wait(&o_staged[qt], 0u, abort_flag, err)) {
#pragma unroll
            for (int c = 0; c < F5_SLICES; ++c)
              tma_store_3d(&tmO, stage + c * (F5_ROWS * 128), c * 64, kh * G, t0 + tok_first);
            tma_store_commit();
            tma_store_wait_read();
          }
        } else
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 64) {
          uint32_t o[2][32];
          t5_ld32_issue(lane_base + 2 * F5_TILE + c0, o[0]);
          t5_ld32_issue(lane_base + 2 * F5_TILE + c0 + 32, o[1]);
          t5_wait_ld();
          if (valid) {
#pragma unroll
            for (int c = 0; c < 64; c += 16) {             // 32 bytes a store: whole sectors
              uint32_t v[8];
#pragma unroll
              for (int e = 0; e < 8; ++e)
                v[e] = pack_bf16(__uint_as_float(o[c >> 5][(c & 31) + 2 * e]) * inv, __uint_as_float(o[c >> 5][(c & 31) + 2 * e + 1]) * inv);
              asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n" ::"l"(orow + c0 + c), "r"(v[0]), "r"(v[1]), "r"(v[2]),
                           "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
            }
          }
        }
      }
    }
  }
  t5_fence_before();
  __syncthreads();
  if (warp == 4 * NQ + 1) t5_dealloc(tmem_base, C::TMEM_COLS);
}

#endif  // VOB_HD == 64 || VOB_HD == 128

}  // namespace vob

using namespace vob;

// Heads in a box of the query's and the output's tensor maps (vob_tensor_map_bf16_heads with boxes of this many heads and
// 128 / this many tokens, rounded down: a tile holds whole tokens), or 0 if this kernel does not take these head counts.
VOB_API int vob_attention_prefill_q_box_heads(int nh, int kvh) {
#if VOB_HD == 64 || VOB_HD == 128
  if (kvh <= 0 || nh % kvh) return 0;
  const int G = nh / kvh;
  return G <= F5_ROWS ? G : 0;
#else
  return 0;
#endif
}

VOB_API int vob_attention_prefill_has_tc5() {
#if VOB_HD == 64 || VOB_HD == 128
  return 1;
#else
  return 0;
#endif
}

// As vob_attention_prefill_tma (same tensor maps: 64-column slices, boxes of vob_attention_decode_box_keys rows), for
// head sizes 64 and 128.  `query_tiles` is 1 or 2: how many tiles of 128 query rows a block takes.
VOB_API int vob_attention_prefill_tc5(const void* map_k, const void* map_v, const void* map_q, const void* map_o, const void* q, long q_stride, void* out,
                                      const int* block_tables, int table_stride, const int* cu_q, const int* context_lens,
                                      int num_requests, int max_q, int nh, int kvh, int block_size, int window, float scale,
                                      long num_pages, int query_tiles, int* err, cudaStream_t stream) {
#if VOB_HD == 64 || VOB_HD == 128
  if (num_requests <= 0 || max_q <= 1) return 0;
  if (!map_k || !map_v) return VOB_BAD_ARGUMENT;
  if (((uintptr_t)out & 31) || ((uintptr_t)q & 15)) return VOB_BAD_ARGUMENT;     // 32-byte stores, 16-byte copies
  if (kvh <= 0 || nh % kvh || block_size <= 0 || block_size % 16 || kvh > 65535 || num_requests > 65535 ||
      (query_tiles != 1 && query_tiles != 2) || !(scale > 0.f))   // the kernel takes maxima before it scales
    return VOB_UNSUPPORTED;
  if (nh / kvh > F5_ROWS) return VOB_UNSUPPORTED;
  const long tiles = ((long)max_q + F5_ROWS / (nh / kvh) - 1) / (F5_ROWS / (nh / kvh));   // tiles of whole tokens
  const int box_keys = block_size % F5_TILE == 0 ? F5_TILE : RUN_KEYS;
  // the query tiles come by TMA when a map was given
  const int q_by_tma = map_q != nullptr && vob_attention_prefill_q_box_heads(nh, kvh) > 0;
  const int o_by_tma = map_o != nullptr && vob_attention_prefill_q_box_heads(nh, kvh) > 0;   // whole output tiles leave the same way
  static bool configured[2] = {false, false};
  if (query_tiles == 1) {
    if (!configured[0]) {
      cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc5_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, F5<1>::SMEM_BYTES);
      if (e != cudaSuccess) return (int)e;
      configured[0] = true;
    }
    dim3 grid((unsigned)tiles * kvh, 1, num_requests);
    return launch_kernel(attention_prefill_tc5_kernel<1>, grid, F5<1>::THREADS, F5<1>::SMEM_BYTES, stream,
                         *(const CUtensorMap*)map_k, *(const CUtensorMap*)map_v, *(const CUtensorMap*)(q_by_tma ? map_q : map_k), q_by_tma,
                         *(const CUtensorMap*)(o_by_tma ? map_o : map_k), o_by_tma,
                         (const __nv_bfloat16*)q, q_stride,
                         (__nv_bfloat16*)out, block_tables, table_stride, cu_q, context_lens, nh, kvh, block_size, window,
                         scale, num_pages, box_keys, err);
  }
  if (!configured[1]) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc5_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, F5<2>::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured[1] = true;
  }
  dim3 grid((unsigned)((tiles + 1) / 2) * kvh, 1, num_requests);
  return launch_kernel(attention_prefill_tc5_kernel<2>, grid, F5<2>::THREADS, F5<2>::SMEM_BYTES, stream,
                       *(const CUtensorMap*)map_k, *(const CUtensorMap*)map_v, *(const CUtensorMap*)(q_by_tma ? map_q : map_k), q_by_tma,
                         *(const CUtensorMap*)(o_by_tma ? map_o : map_k), o_by_tma,
                       (const __nv_bfloat16*)q, q_stride,
                       (__nv_bfloat16*)out, block_tables, table_stride, cu_q, context_lens, nh, kvh, block_size, window,
                       scale, num_pages, box_keys, err);
#else
  return VOB_UNSUPPORTED;
#endif
}
