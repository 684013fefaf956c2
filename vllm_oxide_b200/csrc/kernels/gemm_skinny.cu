// out[M,N] = x[M,K] * W[N,K]^T in bfloat16 for decode-sized batches (M <= 16): a weight-streaming
// kernel.  The time of such a product is the time to read W once, so everything serves that read:
//
//   * persistent blocks (two per SM) walk tiles of 32 rows of W (16 when W has too few rows to give
//     every SM a tile); a producer thread streams each tile, 256 columns per stage, with TMA
//     (cp.async.bulk.tensor through tensor maps: ONE copy of W and one of the tokens per stage, each four
//     column slices of [rows x 64], 128-byte swizzled, completion counted on an mbarrier) into a ring of 4-8 stages, running
//     ahead across tile boundaries, so the copies never stop while the other warps finish a tile; rows
//     and columns beyond the matrices arrive as zeros.  The copy engine moves about 30 bytes per clock
//     and SM, tokens included, so the taller tile matters: it halves the tokens' share of the copies;
//   * four consumer warps share the k-steps of a stage and multiply on tensor cores with W as the
//     16-row operand and the tokens as the 8-wide one (m16n8k16, float accumulation), then sum
//     their partial tiles through shared memory;
//   * the epilogue is fused: round to bfloat16 (plain), or round and widen to float (logits), or
//     SiLU(gate) * up with the gate and up rows of the same eight outputs in one tile, so the
//     [M, 2*intermediate] tensor never exists.  Rounding follows the reference: the product is
//     rounded to bfloat16 once; SiLU is rounded, then the product with `up` is rounded.
//
//   * the residual stream can stay inside the products (decode-sized steps have no other use for the separate
//     add+norm kernel, and every kernel less in the chain of a layer saves about 4 us):
//       - EPI_ADD rounds the product to bfloat16 and adds it to `out` in place: out is the residual stream,
//         so the output product of the attention and the down product leave residual' = x + residual behind;
//       - NORM 1 reads that stream as its tokens and applies RMSNorm on the fly: the consumer warps multiply the
//         token fragments by the norm's weight in registers and sum their squares on the way (a block reads
//         all of K for its tile anyway), and the epilogue scales every sum by 1/sqrt(mean square + eps) of its
//         token, which is the same product up to the place where bfloat16 rounds;
//       - that arithmetic on every fragment of every block costs a product about 2 us, so the product BEFORE can do
//         it once instead: EPI_ADD, given the weight of the norm that follows, also writes bfloat16(stream * weight)
//         to a second buffer and, per tile and token, the sum of the squares of the stream values it wrote;
//         NORM 2 then takes that buffer as its tokens, runs the plain loop, adds the tiles' sums in a fixed order
//         at its start and scales by 1/rms in the epilogue: the same values as NORM 1 up to the order in which
//         the squares are added.
//
// Every wait on an mbarrier is bounded: a wait that runs out sets an error bit and a block-wide
// abort flag; the block then waits (bounded again) for the copies it still has in flight and returns.
#define VOB_TIMEOUT_WHERE 0x100
#include "tensor_map.cuh"


namespace vob {

constexpr int SK_KC = 256;                 // columns per stage
constexpr int SK_SLICES = SK_KC / TMA_BOX_COLS;   // boxes of 64 columns per stage
constexpr int SK_CONSUMERS = 4;
constexpr int SK_THREADS = (SK_CONSUMERS + 1) * 32;

enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_SWIGLU = 2, EPI_ADD = 3 };

__device__ __forceinline__ void sk_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void sk_ldmatrix_x2(uint32_t (&r)[2], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void sk_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// stages of the ring: about 100 KB of shared memory per block, two blocks per SM
#ifndef VOB_SK_RING_KB
#define VOB_SK_RING_KB 96
#endif
template <int R, int MT> struct SkStages { static constexpr int N = (VOB_SK_RING_KB * 1024) / (SK_SLICES * (R + MT) * 128); };

// tmW: W [N, K] with box [R, 64]; tmX: x [M, K] with box [MT, 64].  EPI_BF16 / EPI_F32: out [M, N] (row
// stride ldo).  EPI_SWIGLU: the rows of W alternate in groups of eight between gate and up (gate rows
// 8i..8i+7 of the original at 16i..16i+7, the up rows of the same outputs at 16i+8..16i+15), so every 16
// rows of a tile hold both halves of eight outputs; out [M, N/2].
template <int R, int MT, int EPI, int NORM>
__global__ void __launch_bounds__(SK_THREADS, 2)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, void* out,
                   long ldo, int M, int N, int K, int num_tiles, const float* __restrict__ norm_w, float eps,
                   const float* ss_parts, int ss_count, const float* __restrict__ emit_w, __nv_bfloat16* emit_xn,
                   float* emit_ss, int* err) {
  constexpr int S = SkStages<R, MT>::N;
  constexpr int RT = R / 16, NT = MT / 8;
  constexpr int W_SLICE = R * 128, X_SLICE = MT * 128;
  constexpr int STAGE_BYTES = SK_SLICES * (W_SLICE + X_SLICE);
  extern __shared__ __align__(1024) char smem_raw[];
  char* stages = reinterpret_cast<char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  float* red = reinterpret_cast<float*>(stages + S * STAGE_BYTES);          // [SK_CONSUMERS][R][MT]
  float* sumsq = red + SK_CONSUMERS * R * MT;                                // [SK_CONSUMERS][16] squares of a token, per warp
  uint64_t* full = reinterpret_cast<uint64_t*>(sumsq + SK_CONSUMERS * 16);
  uint64_t* empty = full + S;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + S);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_iters = (K + SK_KC - 1) / SK_KC;
  const unsigned withheld = vob_test_withhold_copies;   // tests of the bounded waits only; read here, used after the set-up
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], SK_CONSUMERS); }
    *abort_flag = 0;
    tma_prefetch_map(&tmW);
    tma_prefetch_map(&tmX);
  }
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  __syncthreads();

  const int m_rows = M < MT ? M : MT;
  pdl_launch_dependents();
  if (warp == SK_CONSUMERS) {
    // ------------------------------------------------ producer (one thread)
    if (lane == 0 && !withheld) {
      const int my_tiles = blockIdx.x < num_tiles ? (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
      const long total = (long)my_tiles * k_iters;
      // The weights do not depend on the kernel before this one: the first stages of W are on their way
      // before that kernel has finished.  The tokens do, so their copies follow the wait.
      const int ahead = total < S ? (int)total : S;
      for (int it0 = 0; it0 < ahead; ++it0) {
        const int tile = blockIdx.x + (it0 / k_iters) * gridDim.x, kc = it0 % k_iters;
        mbar_expect_tx(&full[it0], (unsigned)STAGE_BYTES);
        tma_load_3d(stages + it0 * STAGE_BYTES, &tmW, 0, tile * R, kc * SK_SLICES, &full[it0]);
      }
      pdl_wait();
      for (int it0 = 0; it0 < ahead; ++it0)
        tma_load_3d(stages + it0 * STAGE_BYTES + SK_SLICES * W_SLICE, &tmX, 0, 0, (it0 % k_iters) * SK_SLICES, &full[it0]);
      long it = ahead;
      bool ok = true;
      for (; it < total; ++it) {
        const int tile = blockIdx.x + (int)(it / k_iters) * gridDim.x, kc = (int)(it % k_iters);
        const int s = (int)(it % S);
        ok = mbar_wait(&empty[s], (unsigned)(((it / S) - 1) & 1), abort_flag, err);
        if (!ok) break;
        mbar_expect_tx(&full[s], (unsigned)STAGE_BYTES);
        char* st = stages + s * STAGE_BYTES;
        tma_load_3d(st, &tmW, 0, tile * R, kc * SK_SLICES, &full[s]);
        tma_load_3d(st + SK_SLICES * W_SLICE, &tmX, 0, 0, kc * SK_SLICES, &full[s]);
      }
      // every copy this block issued must have landed before the block may exit
      const long first = it > S ? it - S : 0;
      for (long j = first; j < it; ++j) {
        bool done = false;
        for (unsigned i = 0; i < MBAR_SPIN_LIMIT && !done; ++i) done = mbar_try_wait(&full[j % S], (unsigned)((j / S) & 1));
        if (!done) atomicOr(err, VOB_ERR_TIMEOUT_BITS);
      }
    }
  } else {
    // ------------------------------------------------ consumers
    pdl_wait();   // they write `out`, which the kernel before this one may still read
    if (NORM == 2) {
      // 1/rms of every token from the sums of squares that the product before left per tile: a fixed order of additions
      // (thread t adds the parts t / MT, t / MT + 128 / MT, ... of token t % MT, then one thread a token adds those)
      constexpr int STEP = SK_CONSUMERS * 32 / MT;
      float part = 0.f;
      for (int p = (int)threadIdx.x / MT; p < ss_count; p += STEP) part += ss_parts[(long)p * MT + (int)threadIdx.x % MT];
      red[threadIdx.x] = part;
      asm volatile("bar.sync 1, %0;\n" ::"n"(SK_CONSUMERS * 32) : "memory");
      if ((int)threadIdx.x < MT) {
        float total = 0.f;
#pragma unroll
        for (int q = 0; q < STEP; ++q) total += red[q * MT + threadIdx.x];
        sumsq[threadIdx.x] = 1.f / sqrtf(total / (float)K + eps);
      }
      asm volatile("bar.sync 1, %0;\n" ::"n"(SK_CONSUMERS * 32) : "memory");
    }
    const int g = lane >> 2, tq = lane & 3;
    const int mi = lane >> 3, r8 = lane & 7;
    const int a_row = (mi & 1) * 8 + r8, a_chunk = mi >> 1;                       // W rows, ldmatrix x4
    const int b_row = MT == 16 ? (mi >> 1) * 8 + r8 : r8;                         // token rows, x4 / x2
    const int b_chunk = MT == 16 ? (mi & 1) : ((lane >> 3) & 1);
    long it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      // EPI_ADD: what the tile's outputs hold now, asked for before the products rather than at their end
      constexpr int ADD_PER_THREAD = (R * MT + SK_CONSUMERS * 32 - 1) / (SK_CONSUMERS * 32);
      float prev[ADD_PER_THREAD];
      if (EPI == EPI_ADD) {
#pragma unroll
        for (int i = 0; i < ADD_PER_THREAD; ++i) {
          const int idx = (int)threadIdx.x + i * SK_CONSUMERS * 32;
          const int tok = idx / R;
          const long n = (long)tile * R + idx % R;
          prev[i] = (idx < R * m_rows && n < N) ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(out)[(long)tok * ldo + n]) : 0.f;
        }
      }
      float acc[RT][NT][4];
#pragma unroll
      for (int i = 0; i < RT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
      float ss[2] = {0.f, 0.f};                                  // NORM: squares of tokens g and g + 8 seen by this thread
      for (int kc = 0; kc < k_iters; ++kc, ++it) {
        const int s = (int)(it % S);
        // NORM: the norm's weights for this thread's columns of the stage, asked for before the wait for the stage
        // (they come from L2 and would otherwise stand between every ldmatrix and its mma)
        float2 nw[SK_KC / 16 / SK_CONSUMERS][2];
        if (NORM == 1) {
#pragma unroll
          for (int jj = 0; jj < SK_KC / 16 / SK_CONSUMERS; ++jj) {
            const int k0 = kc * SK_KC + (warp + jj * SK_CONSUMERS) * 16 + tq * 2;
            nw[jj][0] = nw[jj][1] = make_float2(0.f, 0.f);
            if (k0 + 8 < K) {
              nw[jj][0] = __ldg(reinterpret_cast<const float2*>(norm_w + k0));
              nw[jj][1] = __ldg(reinterpret_cast<const float2*>(norm_w + k0 + 8));
            }
          }
        }
        bool ok = mbar_wait(&full[s], (unsigned)((it / S) & 1), abort_flag, err);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const char* st = stages + s * STAGE_BYTES;
        const char* xt = st + SK_SLICES * W_SLICE;
#pragma unroll
        for (int jj = 0; jj < SK_KC / 16 / SK_CONSUMERS; ++jj) {   // columns beyond K are zeros
          const int j = warp + jj * SK_CONSUMERS;
          const int c = j >> 2, ch = (j & 3) * 2;
          uint32_t b[4];
          if (MT == 16) {
            sk_ldmatrix_x4(b, xt + c * X_SLICE + swizzled_offset(b_row, ch + b_chunk));
          } else {
            uint32_t b2[2];
            sk_ldmatrix_x2(b2, xt + c * X_SLICE + swizzled_offset(b_row, ch + b_chunk));
            b[0] = b2[0]; b[1] = b2[1]; b[2] = b[3] = 0;
          }
          if (NORM == 1) {
            // b[0], b[1]: token g at columns k, k+1 and k+8, k+9 of this 16-column step; b[2], b[3]: token g + 8
            const float2 w0 = nw[jj][0], w1 = nw[jj][1];
#pragma unroll
            for (int r = 0; r < (MT == 16 ? 4 : 2); ++r) {
              const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b[r]));
              ss[r >> 1] = fmaf(v.x, v.x, fmaf(v.y, v.y, ss[r >> 1]));
              const float2 wv = (r & 1) ? w1 : w0;
              const __nv_bfloat162 scaled = __floats2bfloat162_rn(v.x * wv.x, v.y * wv.y);
              b[r] = *reinterpret_cast<const uint32_t*>(&scaled);
            }
          }
#pragma unroll
          for (int i = 0; i < RT; ++i) {
            uint32_t a[4];
            sk_ldmatrix_x4(a, st + c * W_SLICE + swizzled_offset(i * 16 + a_row, ch + a_chunk));
            sk_mma(acc[i][0], a, b[0], b[1]);
            if (MT == 16) sk_mma(acc[i][NT - 1], a, b[2], b[3]);
          }
        }
        // The stage goes back to the copy engine.  What this warp read of it with ordinary loads (ldmatrix) is ordered
        // before the engine's next write only across a proxy fence: without it a refill that came fast (the matrix in
        // L2, a block with several tiles) overwrote a stage that was still being read.
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
      }
      if (NORM == 1) {
        // the four lanes of a token hold different columns: add them, then one lane writes the warp's share
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          ss[h] += __shfl_xor_sync(0xffffffffu, ss[h], 1);
          ss[h] += __shfl_xor_sync(0xffffffffu, ss[h], 2);
        }
        if (tq == 0) { sumsq[warp * 16 + g] = ss[0]; sumsq[warp * 16 + 8 + g] = ss[1]; }
      }
      // sum the four warps' partial tiles (a warp whose wait ran out still meets the others at the barriers)
#pragma unroll
      for (int i = 0; i < RT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          float* p0 = red + ((warp * R + i * 16 + g) * MT) + j * 8 + tq * 2;
          float* p1 = red + ((warp * R + i * 16 + g + 8) * MT) + j * 8 + tq * 2;
          p0[0] = acc[i][j][0]; p0[1] = acc[i][j][1];
          p1[0] = acc[i][j][2]; p1[1] = acc[i][j][3];
        }
      asm volatile("bar.sync 1, %0;\n" ::"n"(SK_CONSUMERS * 32) : "memory");
      const int tid = threadIdx.x;
      const bool aborted = *abort_flag != 0;
      if (aborted) {
        // nothing is written for a tile that was not finished
      } else if (EPI == EPI_SWIGLU) {
        for (int idx = tid; idx < (R / 2) * m_rows; idx += SK_CONSUMERS * 32) {
          const int tok = idx / (R / 2), r = idx % (R / 2);
          const long n = (long)tile * (R / 2) + r;
          if (n >= N / 2) continue;
          const int gr = (r >> 3) * 16 + (r & 7);       // gate row in the tile; its up row is 8 further
          float gate = 0.f, up = 0.f;
#pragma unroll
          for (int w = 0; w < SK_CONSUMERS; ++w) { gate += red[(w * R + gr) * MT + tok]; up += red[(w * R + gr + 8) * MT + tok]; }
          if (NORM) {
            const float inv = NORM == 2 ? sumsq[tok]
                                        : 1.f / sqrtf((sumsq[tok] + sumsq[16 + tok] + sumsq[32 + tok] + sumsq[48 + tok]) / (float)K + eps);
            gate *= inv;
            up *= inv;
          }
          gate = bf16_round(gate);
          up = bf16_round(up);
          const float act = bf16_round(gate / (1.f + expf(-gate)));
          reinterpret_cast<__nv_bfloat16*>(out)[(long)tok * ldo + n] = __float2bfloat16_rn(act * up);
        }
      } else {
#pragma unroll
        for (int i = 0; i < ADD_PER_THREAD; ++i) {
          const int idx = tid + i * SK_CONSUMERS * 32;
          const int tok = idx / R, r = idx % R;
          const long n = (long)tile * R + r;
          float sq = 0.f;                                  // EPI_ADD with emit: the square of the stream value written here
          if (idx < R * m_rows && n < N) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < SK_CONSUMERS; ++w) v += red[(w * R + r) * MT + tok];
            if (NORM == 1) v *= 1.f / sqrtf((sumsq[tok] + sumsq[16 + tok] + sumsq[32 + tok] + sumsq[48 + tok]) / (float)K + eps);
            if (NORM == 2) v *= sumsq[tok];
            if (EPI == EPI_F32) {
              reinterpret_cast<float*>(out)[(long)tok * ldo + n] = bf16_round(v);
            } else if (EPI == EPI_ADD) {
              const float sv = bf16_round(bf16_round(v) + prev[i]);
              reinterpret_cast<__nv_bfloat16*>(out)[(long)tok * ldo + n] = __float2bfloat16_rn(sv);
              if (emit_xn) {
                emit_xn[(long)tok * N + n] = __float2bfloat16_rn(sv * __ldg(emit_w + n));
                sq = sv * sv;
              }
            } else {
              reinterpret_cast<__nv_bfloat16*>(out)[(long)tok * ldo + n] = __float2bfloat16_rn(v);
            }
          }
          if (EPI == EPI_ADD && emit_ss) {                  // the same for every thread of the block
            // the R lanes that hold a token's rows of this tile add their squares; tokens beyond the batch give 0
#pragma unroll
            for (int o = R / 2; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            if (r == 0 && tok < MT) emit_ss[(long)tile * MT + tok] = sq;
          }
        }
      }
      asm volatile("bar.sync 1, %0;\n" ::"n"(SK_CONSUMERS * 32) : "memory");
      if (aborted) break;
    }
  }
  __syncthreads();
}

struct SkExtra {        // what only some products use
  const float* ss_parts = nullptr;   // NORM 2: [ss_count][MT] sums of squares of the tokens, per tile of the product before
  int ss_count = 0;
  const float* emit_w = nullptr;     // EPI_ADD: weight [N] of the norm that follows,
  __nv_bfloat16* emit_xn = nullptr;  //          where bfloat16(stream * weight) goes, [M, N],
  float* emit_ss = nullptr;          //          and the sums of squares, [tiles][MT]
};

template <int R, int MT, int EPI, int NORM>
static int skinny_launch(const CUtensorMap* tmW, const CUtensorMap* tmX, void* out, long ldo, int M, int N, int K,
                         const float* norm_w, float eps, const SkExtra& x, int* err, cudaStream_t stream) {
  constexpr int S = SkStages<R, MT>::N;
  const int smem = 1024 + S * SK_SLICES * (R + MT) * 128 + SK_CONSUMERS * (R * MT + 16) * (int)sizeof(float) + 2 * S * 8 + 16;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<R, MT, EPI, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int num_tiles = (N + R - 1) / R;
  const int resident = 2 * sm_count();   // two blocks of this kernel fit an SM
  const int grid = num_tiles < resident ? num_tiles : resident;
  return launch_kernel(gemm_skinny_kernel<R, MT, EPI, NORM>, grid, SK_THREADS, smem, stream, *tmW, *tmX, out, ldo, M, N, K,
                       num_tiles, norm_w, eps, x.ss_parts, x.ss_count, x.emit_w, x.emit_xn, x.emit_ss, err);
}

template <int R, int MT>
static int skinny_dispatch(int epilogue, const CUtensorMap* tw, const CUtensorMap* tx, void* out, long ldo, int M, int N,
                           int K, const float* norm_w, float eps, const SkExtra& x, int* err, cudaStream_t stream) {
  if (x.ss_parts) {   // the tokens come already multiplied by the norm's weight; 1/rms from the sums the product before left
    if (epilogue == EPI_BF16) return skinny_launch<R, MT, EPI_BF16, 2>(tw, tx, out, ldo, M, N, K, nullptr, eps, x, err, stream);
    if (epilogue == EPI_SWIGLU) return skinny_launch<R, MT, EPI_SWIGLU, 2>(tw, tx, out, ldo, M, N, K, nullptr, eps, x, err, stream);
    return VOB_UNSUPPORTED;
  }
  if (norm_w) {   // the norm in front is instantiated for the two products that follow a norm in a layer
    if (epilogue == EPI_BF16) return skinny_launch<R, MT, EPI_BF16, 1>(tw, tx, out, ldo, M, N, K, norm_w, eps, x, err, stream);
    if (epilogue == EPI_SWIGLU) return skinny_launch<R, MT, EPI_SWIGLU, 1>(tw, tx, out, ldo, M, N, K, norm_w, eps, x, err, stream);
    return VOB_UNSUPPORTED;
  }
  if (epilogue == EPI_BF16) return skinny_launch<R, MT, EPI_BF16, 0>(tw, tx, out, ldo, M, N, K, nullptr, 0.f, x, err, stream);
  if (epilogue == EPI_F32) return skinny_launch<R, MT, EPI_F32, 0>(tw, tx, out, ldo, M, N, K, nullptr, 0.f, x, err, stream);
  if (epilogue == EPI_SWIGLU) return skinny_launch<R, MT, EPI_SWIGLU, 0>(tw, tx, out, ldo, M, N, K, nullptr, 0.f, x, err, stream);
  if (epilogue == EPI_ADD) return skinny_launch<R, MT, EPI_ADD, 0>(tw, tx, out, ldo, M, N, K, nullptr, 0.f, x, err, stream);
  return VOB_BAD_ARGUMENT;
}

}  // namespace vob

using namespace vob;

// For tests of the bounded waits: the number of tries after which a pipeline wait of this kernel gives up (0: the
// default), and whether the producers withhold their copies.  With the copies withheld every block's first wait is for
// something that never comes: after `tries` attempts the blocks set VOB_ERR_TIMEOUT | VOB_WHERE_GEMM_SKINNY in the error
// word, write nothing and return (nothing is in flight).  Takes effect for launches made after it on the current device.
VOB_API int vob_gemm_skinny_set_wait_limit(unsigned tries, int withhold_copies) {
  return set_wait_limit(tries, withhold_copies ? 1u : 0u);
}

// Box rows the weight map must have for a matrix of N rows: 32, or 16 when 32-row tiles would leave SMs idle.
VOB_API int vob_gemm_skinny_weight_box(long N) { return (N + 31) / 32 >= vob::sm_count() ? 32 : 16; }

// Box rows the token map must have for a batch of M rows.
VOB_API int vob_gemm_skinny_token_box(int M) { return M <= 8 ? 8 : 16; }

// map_w: tensor map of W [N, K] with box rows vob_gemm_skinny_weight_box(N); map_x: tensor map of x [M, K] with box
// rows vob_gemm_skinny_token_box(M) (both from vob_tensor_map_bf16_sliced with 4 slices per box, host memory; K must be
// a multiple of 64).
// epilogue: 0 bfloat16 out [M,N]; 1 float out [M,N] (rounded to bfloat16 first); 2 SiLU(gate)*up over rows that
// alternate in groups of eight between gate and up, out [M,N/2] bfloat16; 3 out [M,N] bfloat16 += the product rounded to
// bfloat16 (the residual stream).  norm_w (may be null; epilogues 0 and 2): float [K], the weight of an RMSNorm with
// `eps` that is applied to x on the way.  ss_parts (may be null; instead of norm_w): x is already the tokens times the
// norm's weight, and ss_parts [ss_count][8 or 16] (the token rows of a box for this M) holds sums of squares of the
// unscaled tokens that add up to each token's; the product is scaled by 1/rms.  emit_w / emit_xn / emit_ss (all or none;
// epilogue 3): beside the sum into `out`, bfloat16(out * emit_w) goes to emit_xn [M, N] and, per tile of
// vob_gemm_skinny_weight_box(N) rows and token, the sum of the squares of the new values of `out` to emit_ss.  Needs M <= 16.
VOB_API int vob_gemm_skinny(const void* map_w, const void* map_x, void* out, long ldo, int M, int N, int K, int epilogue,
                            const float* norm_w, float eps, const float* ss_parts, int ss_count, const float* emit_w,
                            void* emit_xn, float* emit_ss, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 16 || K <= 0 || K % 64 || !map_w || !map_x) return VOB_UNSUPPORTED;
  if (epilogue == EPI_SWIGLU && N % 16) return VOB_BAD_ARGUMENT;
  if (norm_w && (uintptr_t)norm_w % 8) return VOB_BAD_ARGUMENT;
  if (ss_parts && (norm_w || ss_count <= 0)) return VOB_BAD_ARGUMENT;
  if ((emit_w != nullptr) != (emit_xn != nullptr) || (emit_w != nullptr) != (emit_ss != nullptr)) return VOB_BAD_ARGUMENT;
  if (emit_w && epilogue != EPI_ADD) return VOB_BAD_ARGUMENT;
  SkExtra x;
  x.ss_parts = ss_parts; x.ss_count = ss_count;
  x.emit_w = emit_w; x.emit_xn = (__nv_bfloat16*)emit_xn; x.emit_ss = emit_ss;
  const CUtensorMap* tw = (const CUtensorMap*)map_w;
  const CUtensorMap* tx = (const CUtensorMap*)map_x;
  const bool tall = vob_gemm_skinny_weight_box(N) == 32;
  if (M <= 8) return tall ? skinny_dispatch<32, 8>(epilogue, tw, tx, out, ldo, M, N, K, norm_w, eps, x, err, stream)
                          : skinny_dispatch<16, 8>(epilogue, tw, tx, out, ldo, M, N, K, norm_w, eps, x, err, stream);
  return tall ? skinny_dispatch<32, 16>(epilogue, tw, tx, out, ldo, M, N, K, norm_w, eps, x, err, stream)
              : skinny_dispatch<16, 16>(epilogue, tw, tx, out, ldo, M, N, K, norm_w, eps, x, err, stream);
}
