// out[M,N] = x[M,K] * W[N,K]^T in bfloat16 for steps of 17 to 128 tokens (decoding at larger batch sizes,
// short portions), on the fifth-generation tensor cores: tcgen05.mma with the accumulator in tensor memory.
//
// Such a product still costs the time to read W once, so the weights are the 128-row operand ("swap-AB"):
// a tile is 128 rows of W against all tokens of the step (padded to 32, 64 or 128), D[128 x tokens] in float
// lives in TMEM, and every byte of W is read exactly once.  One block per SM walks the tiles:
//   warp 0      producer: per 64 columns of K one TMA copy of the W tile [128 x 64] and one of the tokens
//               [tokens x 64] (128-byte swizzle) into a ring of stages;
//   warp 1      allocates TMEM (two accumulators) and issues the MMAs: four tcgen05.mma (K = 16 each) per
//               stage from shared-memory descriptors; tcgen05.commit hands a stage back to the producer and,
//               after the last one of a tile, the accumulator to the epilogue;
//   warps 2-5   epilogue: tcgen05.ld brings the accumulator to registers (a thread owns one row of W, that is
//               one output feature, for all tokens), rounds, and stores; the next tile's MMAs run meanwhile
//               into the other accumulator.
// A matrix with few 128-row tiles (or a number of tiles that fills the last round of blocks badly) is also
// split along K: a unit of work is (tile, K range); its float partial tile goes to scratch memory, a counter
// per tile tells the last unit to finish that it is the last, and that one sums the partials in a fixed order and
// runs the epilogue (and sets the counter back to zero for the next launch).
// Epilogues as in the weight-streaming kernel for smaller steps: bfloat16, float logits, SiLU(gate)*up over
// interleaved gate/up rows.  Every wait on an mbarrier is bounded; on a timeout the block sets an error bit,
// stops issuing work, and still frees its TMEM before it returns.
#include "tcgen05.cuh"

namespace vob {

constexpr int T5_ROWS = 128;      // rows of W per tile (the MMA's M)
constexpr int T5_KC = 64;         // columns of K per stage: one 128-byte swizzle atom
constexpr int T5_THREADS = 192;
constexpr int T5_EPI_WARPS = 4;

enum { T5_EPI_BF16 = 0, T5_EPI_F32 = 1, T5_EPI_SWIGLU = 2 };

__device__ __forceinline__ float t5_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <int NT> struct T5Stages { static constexpr int N = (192 * 1024) / ((T5_ROWS + NT) * 128); };

// tmW: W [N, K] as 2-D map with box [128 rows, 64 columns]; tmX: x [M, K] with box [NT rows, 64 columns].
template <int NT, int EPI>
__global__ void __launch_bounds__(T5_THREADS, 1)
gemm_tc5_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, void* __restrict__ out,
                long ldo, int M, int N, int K, int num_tiles, int ksplit, int kb_per_split, float* __restrict__ partials,
                int* __restrict__ counters, int* err) {
  constexpr int S = T5Stages<NT>::N > 8 ? 8 : T5Stages<NT>::N;
  constexpr int A_BYTES = T5_ROWS * 128, B_BYTES = NT * 128, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = 2 * NT < 32 ? 32 : 2 * NT;      // two accumulators; a power of two
  extern __shared__ __align__(1024) char smem_raw[];
  char* stages = reinterpret_cast<char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(stages + S * STAGE_BYTES);
  uint64_t* empty = full + S;
  uint64_t* acc_full = empty + S;       // [2] MMA -> epilogue
  uint64_t* acc_empty = acc_full + 2;   // [2] epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_iters = (K + T5_KC - 1) / T5_KC;
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], T5_EPI_WARPS); }
    *abort_flag = 0;
    tma_prefetch_map(&tmW);
    tma_prefetch_map(&tmX);
  }
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  if (warp == 1) {   // one warp allocates the tensor memory for the block and publishes its address
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  t5_fence_before();
  __syncthreads();
  t5_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  // a unit of work is (tile, K range): unit u covers tile u / ksplit and stages [ks * kb_per_split, ...) of K
  const int num_units = num_tiles * ksplit;
  const int my_units = (int)blockIdx.x < num_units ? (num_units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  auto unit_kb0 = [&](int u) { return (u % ksplit) * kb_per_split; };
  auto unit_kbn = [&](int u) { const int b = (u % ksplit) * kb_per_split; return min(k_iters, b + kb_per_split) - b; };

  if (warp == 0) {
    // ------------------------------------------------ producer (one thread)
    if (lane == 0) {
      // W does not depend on the kernel before this one: its first stages are on their way before that kernel ends
      long it = 0;
      int lu = 0, kb = 0;                              // local unit index and stage within it
      int unit = blockIdx.x;
      auto advance = [&]() { if (++kb >= unit_kbn(unit)) { kb = 0; ++lu; unit += gridDim.x; } };
      int ahead_unit[8], ahead_kb[8], ahead = 0;
      while (ahead < S && lu < my_units) {
        ahead_unit[ahead] = unit; ahead_kb[ahead] = unit_kb0(unit) + kb;
        mbar_expect_tx(&full[ahead], (unsigned)STAGE_BYTES);
        tma_load_2d(stages + ahead * STAGE_BYTES, &tmW, ahead_kb[ahead] * T5_KC, (unit / ksplit) * T5_ROWS, &full[ahead]);
        ++ahead; ++it; advance();
      }
      pdl_wait();
      for (int i = 0; i < ahead; ++i)
        tma_load_2d(stages + i * STAGE_BYTES + A_BYTES, &tmX, ahead_kb[i] * T5_KC, 0, &full[i]);
      for (; lu < my_units; ++it, advance()) {
        const int s = (int)(it % S);
        if (!mbar_wait(&empty[s], (unsigned)(((it / S) - 1) & 1), abort_flag, err)) break;
        const int col = (unit_kb0(unit) + kb) * T5_KC;
        mbar_expect_tx(&full[s], (unsigned)STAGE_BYTES);
        tma_load_2d(stages + s * STAGE_BYTES, &tmW, col, (unit / ksplit) * T5_ROWS, &full[s]);
        tma_load_2d(stages + s * STAGE_BYTES + A_BYTES, &tmX, col, 0, &full[s]);
      }
      const long first = it > S ? it - S : 0;       // copies in flight must land before the block exits
      for (long j = first; j < it; ++j) {
        bool done = false;
        for (unsigned i = 0; i < MBAR_SPIN_LIMIT && !done; ++i) done = mbar_try_wait(&full[j % S], (unsigned)((j / S) & 1));
        if (!done) atomicOr(err, VOB_ERR_TIMEOUT);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer (one thread)
    if (lane == 0) {
      const uint32_t idesc = t5_instr_desc(T5_ROWS, NT);
      long it = 0;
      bool ok = true;
      for (int lt = 0; lt < my_units && ok; ++lt) {
        const int a = lt & 1;
        const int n_kb = unit_kbn(blockIdx.x + lt * gridDim.x);
        if (lt >= 2) {   // the epilogue must have drained this accumulator (two tiles ago)
          ok = mbar_wait(&acc_empty[a], (unsigned)(((lt >> 1) - 1) & 1), abort_flag, err);
          if (!ok) break;
          t5_fence_after();
        }
        const uint32_t d_tmem = tmem_base + (uint32_t)(a * NT);
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int s = (int)(it % S);
          ok = mbar_wait(&full[s], (unsigned)((it / S) & 1), abort_flag, err);
          if (!ok) break;
          t5_fence_after();
          const char* st = stages + s * STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < T5_KC / 16; ++k)      // 16 columns = 32 bytes further into the swizzle atom
            t5_mma(d_tmem, t5_smem_desc(st + k * 32), t5_smem_desc(st + A_BYTES + k * 32), idesc, (kb | k) ? 1u : 0u);
          t5_commit(&empty[s]);                      // the stage is free once these MMAs have read it
        }
        if (ok) t5_commit(&acc_full[a]);             // the accumulator is complete once they have all finished
      }
    }
  } else {
    // ------------------------------------------------ epilogue: warp w reads TMEM lanes 32*(w%4) .. +31
    pdl_wait();   // `out` may still be read by the kernel before this one
    const int q = warp & 3;
    const int m_rows = M < NT ? M : NT;
    for (int lt = 0; lt < my_units; ++lt) {
      const int unit = blockIdx.x + lt * gridDim.x;
      const int tile = unit / ksplit;
      const int a = lt & 1;
      bool ok = mbar_wait(&acc_full[a], (unsigned)((lt >> 1) & 1), abort_flag, err);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      t5_fence_after();
      const int row = q * 32 + lane;                              // this thread's row of the tile
      const long n = (long)tile * T5_ROWS + row;                  // one output feature
      bool finish = true;                                         // whether this unit runs the epilogue
      if (ksplit > 1) {
        // park the partial tile ([token][row]: a warp writes 128 contiguous bytes), hand the accumulator back,
        // and find out whether the other K ranges of this tile are done
        float* mine = partials + (size_t)unit * NT * T5_ROWS;
#pragma unroll
        for (int c0 = 0; c0 < NT; c0 += 32) {
          float v[32];
          t5_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * NT + c0), v);
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c0 + j < m_rows) mine[(size_t)(c0 + j) * T5_ROWS + row] = v[j];
        }
        t5_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[a]);
        // each warp owns 32 rows of the tile and counts per (tile, quarter): no block-wide barrier is needed
        __threadfence();
        __syncwarp();
        int last = 0;
        if (lane == 0) last = atomicAdd(&counters[tile * 4 + q], 1) == ksplit - 1;
        finish = __shfl_sync(0xffffffffu, last, 0) != 0;
        if (finish) __threadfence();
      }
      if (finish) {
#pragma unroll
        for (int c0 = 0; c0 < NT; c0 += 32) {
          if (c0 >= m_rows) break;
          float v[32];
          if (ksplit > 1) {
            // K ranges in ascending order; the 32 loads of a range are independent and in flight together
            const float* base = partials + (size_t)tile * ksplit * NT * T5_ROWS + (size_t)c0 * T5_ROWS + row;
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
            for (int ks = 0; ks < ksplit; ++ks) {
              float t[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) t[j] = c0 + j < m_rows ? __ldcg(base + ((size_t)ks * NT + j) * T5_ROWS) : 0.f;
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] += t[j];
            }
          } else {
            t5_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * NT + c0), v);
          }
          if (EPI == T5_EPI_SWIGLU) {
            // rows alternate in groups of eight between gate and up: lane l (l & 8 == 0) holds a gate row, lane l + 8 its up row
            const long n_out = (long)tile * (T5_ROWS / 2) + q * 16 + (lane >> 4) * 8 + (lane & 7);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float up = __shfl_down_sync(0xffffffffu, v[j], 8);
              const int tok = c0 + j;
              if ((lane & 8) == 0 && tok < m_rows && n_out < N / 2) {
                const float g = t5_round(v[j]);
                const float act = t5_round(g / (1.f + expf(-g)));
                reinterpret_cast<__nv_bfloat16*>(out)[(long)tok * ldo + n_out] = __float2bfloat16_rn(act * t5_round(up));
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int tok = c0 + j;
              if (tok < m_rows && n < N) {
                if (EPI == T5_EPI_F32) reinterpret_cast<float*>(out)[(long)tok * ldo + n] = t5_round(v[j]);
                else reinterpret_cast<__nv_bfloat16*>(out)[(long)tok * ldo + n] = __float2bfloat16_rn(v[j]);
              }
            }
          }
        }
        if (ksplit > 1 && lane == 0) counters[tile * 4 + q] = 0;          // ready for the next launch
      }
      if (ksplit == 1) {
        t5_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[a]);
      }
    }
  }
  // every path ends here: the tensor memory goes back before the block exits
  t5_fence_before();
  __syncthreads();
  if (warp == 1) {
    t5_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

template <int NT, int EPI>
static int tc5_launch(const CUtensorMap* tmW, const CUtensorMap* tmX, void* out, long ldo, int M, int N, int K, int ksplit,
                      float* partials, int* counters, int* err, cudaStream_t stream) {
  constexpr int S = T5Stages<NT>::N > 8 ? 8 : T5Stages<NT>::N;
  const int smem = 1024 + S * (T5_ROWS + NT) * 128 + (2 * S + 4) * 8 + 16;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc5_kernel<NT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int num_tiles = (N + T5_ROWS - 1) / T5_ROWS;
  const int k_iters = (K + T5_KC - 1) / T5_KC;
  const int kb_per_split = (k_iters + ksplit - 1) / ksplit;
  if ((ksplit - 1) * kb_per_split >= k_iters) return VOB_BAD_ARGUMENT;      // a K range would be empty
  const int units = num_tiles * ksplit;
  const int grid = units < 148 ? units : 148;
  return launch_kernel(gemm_tc5_kernel<NT, EPI>, grid, T5_THREADS, smem, stream, *tmW, *tmX, out, ldo, M, N, K, num_tiles,
                       ksplit, kb_per_split, partials, counters, err);
}

template <int NT>
static int tc5_dispatch(int epilogue, const CUtensorMap* tw, const CUtensorMap* tx, void* out, long ldo, int M, int N, int K,
                        int ksplit, float* partials, int* counters, int* err, cudaStream_t stream) {
  if (epilogue == T5_EPI_BF16) return tc5_launch<NT, T5_EPI_BF16>(tw, tx, out, ldo, M, N, K, ksplit, partials, counters, err, stream);
  if (epilogue == T5_EPI_F32) return tc5_launch<NT, T5_EPI_F32>(tw, tx, out, ldo, M, N, K, ksplit, partials, counters, err, stream);
  if (epilogue == T5_EPI_SWIGLU) return tc5_launch<NT, T5_EPI_SWIGLU>(tw, tx, out, ldo, M, N, K, ksplit, partials, counters, err, stream);
  return VOB_BAD_ARGUMENT;
}

}  // namespace vob

using namespace vob;

// Rows of the token box for a step of M tokens (32, 64 or 128).
VOB_API int vob_gemm_tc5_token_box(int M) { return M <= 32 ? 32 : (M <= 64 ? 64 : 128); }

// How many K ranges a product [*, K] x [N, K]^T is split into: the fewest (each at least 512 columns) with which the
// units of work fill the rounds of 148 blocks to 85 % or more; 1 when none does better than no split.
VOB_API int vob_gemm_tc5_ksplit(long N, long K) {
  const long tiles = (N + T5_ROWS - 1) / T5_ROWS, k_iters = (K + T5_KC - 1) / T5_KC;
  double best_eff = 0.0;
  int best = 1;
  for (int ks = 1; ks <= 16; ++ks) {
    const long per = (k_iters + ks - 1) / ks;
    if (ks > 1 && (per * T5_KC < 512 || (ks - 1) * per >= k_iters)) continue;
    const long units = tiles * ks, rounds = (units + 147) / 148;
    const double eff = (double)units / (double)(rounds * 148);
    if (eff >= 0.85) return ks;
    if (eff > best_eff + 1e-9) { best_eff = eff; best = ks; }
  }
  return best;
}

// Floats of scratch for the partial tiles, and counters (ints, zero before the first launch; the kernel leaves them zero).
VOB_API long vob_gemm_tc5_scratch_floats(int M, long N, int ksplit) {
  return ksplit > 1 ? ((N + T5_ROWS - 1) / T5_ROWS) * ksplit * (long)vob_gemm_tc5_token_box(M) * T5_ROWS : 0;
}
VOB_API long vob_gemm_tc5_counters(long N) { return 4 * ((N + T5_ROWS - 1) / T5_ROWS); }

// map_w: vob_tensor_map_bf16_2d of W [N, K] with box rows 128; map_x: of x [M, K] with box rows
// vob_gemm_tc5_token_box(M).  epilogue: 0 bfloat16 out [M,N]; 1 float out [M,N] (rounded to bfloat16 first);
// 2 SiLU(gate)*up over rows that alternate in groups of eight between gate and up, out [M,N/2].  Needs M <= 128.
// ksplit > 1 needs `partials` (vob_gemm_tc5_scratch_floats) and `counters` (vob_gemm_tc5_counters, zeroed).
VOB_API int vob_gemm_tc5(const void* map_w, const void* map_x, void* out, long ldo, int M, int N, int K, int epilogue,
                         int ksplit, float* partials, int* counters, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 128 || K <= 0 || K % 8 || !map_w || !map_x || ksplit < 1) return VOB_UNSUPPORTED;
  if (ksplit > 1 && (!partials || !counters)) return VOB_BAD_ARGUMENT;
  if (epilogue == T5_EPI_SWIGLU && N % 16) return VOB_BAD_ARGUMENT;
  const CUtensorMap* tw = (const CUtensorMap*)map_w;
  const CUtensorMap* tx = (const CUtensorMap*)map_x;
  if (M <= 32) return tc5_dispatch<32>(epilogue, tw, tx, out, ldo, M, N, K, ksplit, partials, counters, err, stream);
  if (M <= 64) return tc5_dispatch<64>(epilogue, tw, tx, out, ldo, M, N, K, ksplit, partials, counters, err, stream);
  return tc5_dispatch<128>(epilogue, tw, tx, out, ldo, M, N, K, ksplit, partials, counters, err, stream);
}
