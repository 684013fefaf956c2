// out[M,N] = x[M,K] * W[N,K]^T in bfloat16 for steps of 17 to 128 tokens (decoding at larger batch sizes,
// short portions), on the fifth-generation tensor cores: tcgen05.mma with the accumulator in tensor memory.
//
// Such a product still costs the time to read W once, so the weights are the 128-row operand ("swap-AB"):
// a tile is 128 rows of W against all tokens of the step (padded to 32, 64 or 128), D[128 x tokens] in float
// lives in TMEM, and every byte of W is read exactly once.  One block per SM (two smaller ones for a matrix of
// between one and two tiles per SM, so that all its tiles are at work at once):
//   warp 0      producer: per 64 columns of K one TMA copy of the W tile [128 x 64] and one of the tokens
//               [tokens x 64] (128-byte swizzle) into a ring of stages; the first W copies are issued before
//               anything else in the block is set up, and before the kernel ahead in the stream has finished;
//   warp 1      allocates TMEM (two accumulators) and issues the MMAs: four tcgen05.mma (K = 16 each) per
//               stage from shared-memory descriptors; tcgen05.commit hands a stage back to the producer and,
//               after the last one of a tile, the accumulator to the epilogue;
//   warps 2-5   epilogue: tcgen05.ld brings the accumulator to registers (a thread owns one row of W, that is
//               one output feature, for all tokens), rounds, and stores; the next tile's MMAs run meanwhile
//               into the other accumulator.
// A matrix with few 128-row tiles is also split along K, over the blocks of a thread-block cluster: the blocks
// of a cluster work on the same tile, block r on the r-th range of K.  Their partial tiles never go to global
// memory: the tokens of the tile are dealt out to the blocks, every block stores its partial values for a token
// into the shared memory of that token's owner (st.shared::cluster), tells the owner through an mbarrier, and
// the owner adds the partials in the order of the ranges and runs the epilogue for its tokens.  A second mbarrier
// tells the writers that the owner has read its buffer, before they fill it for the next tile.
// Epilogues as in the weight-streaming kernel for smaller steps: bfloat16, float logits, SiLU(gate)*up over
// interleaved gate/up rows.  Every wait on an mbarrier is bounded; on a timeout the block sets an error bit,
// stops issuing work, and still frees its TMEM before it returns; the blocks of a cluster leave together, so
// none is signalled after it has gone.
#define VOB_TIMEOUT_WHERE 0x200
#include "tcgen05.cuh"

namespace vob {

constexpr int T5_ROWS = 128;      // rows of W per tile (the MMA's M)
constexpr int T5_KC = 64;         // columns of K per stage: one 128-byte swizzle atom
constexpr int T5_THREADS = 192;
constexpr int T5_EPI_WARPS = 4;
constexpr int T5_MAX_CLUSTER = 8;

enum { T5_EPI_BF16 = 0, T5_EPI_F32 = 1, T5_EPI_SWIGLU = 2 };

__device__ __forceinline__ float t5_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// Shared memory of a block: the ring of stages, then the buffer the cluster's partial tiles are exchanged in
// (blocks x tokens-per-block x 128 floats, at most NT + 7 token rows), then the barriers.  OCC = 2 is the layout for
// two blocks per SM: a shorter ring and no exchange buffer (such blocks never form clusters).
template <int NT, int OCC> struct T5Cfg {
  static constexpr int STAGE_BYTES = (T5_ROWS + NT) * 128;
  static constexpr int XBUF_BYTES = OCC == 1 ? (NT + T5_MAX_CLUSTER) * T5_ROWS * 4 : 0;
  static constexpr int S_FIT = ((OCC == 1 ? 220 : 111) * 1024 - XBUF_BYTES) / STAGE_BYTES;
  static constexpr int S = S_FIT > 8 ? 8 : S_FIT;
  static constexpr int NUM_BARRIERS = 2 * S + 4 + 2 * T5_EPI_WARPS;
  static constexpr int SMEM = 1024 + S * STAGE_BYTES + XBUF_BYTES + NUM_BARRIERS * 8 + 16;
};

__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(a) : "r"(local_smem_addr), "r"(rank));
  return a;
}
__device__ __forceinline__ void store_remote_f32(uint32_t cluster_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(cluster_addr), "f"(v) : "memory");
}
// One arrival on an mbarrier of a block of this cluster; what this thread wrote (and what it has synchronised with) is
// visible to who waits with mbar_wait_cluster.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, unsigned parity, volatile int* abort_flag, int* err) {
  const unsigned addr = smem_addr(bar);
  for (unsigned i = 0; i < MBAR_SPIN_LIMIT; ++i) {
    unsigned ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
    if (ok) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  atomicOr(err, VOB_ERR_TIMEOUT_BITS);
  return false;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

// tmW: W [N, K] as 2-D map with box [128 rows, 64 columns]; tmX: x [M, K] with box [NT rows, 64 columns].
// The grid is (clusters x csize) blocks in clusters of csize; cluster c works on tiles c, c + clusters, ...
template <int NT, int EPI, int OCC>
__global__ void __launch_bounds__(T5_THREADS, OCC)
gemm_tc5_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, void* out,
                long ldo, int M, int N, int K, int num_tiles, int csize, int kb_per_split, int* err) {
  using Cfg = T5Cfg<NT, OCC>;
  constexpr int S = Cfg::S;
  constexpr int A_BYTES = T5_ROWS * 128, STAGE_BYTES = Cfg::STAGE_BYTES;
  constexpr int TMEM_COLS = 2 * NT < 32 ? 32 : 2 * NT;      // two accumulators; a power of two
  extern __shared__ __align__(1024) char smem_raw[];
  char* stages = reinterpret_cast<char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  float* xbuf = reinterpret_cast<float*>(stages + S * STAGE_BYTES);
  uint64_t* full = reinterpret_cast<uint64_t*>(stages + S * STAGE_BYTES + Cfg::XBUF_BYTES);
  uint64_t* empty = full + S;
  uint64_t* acc_full = empty + S;       // [2] MMA -> epilogue
  uint64_t* acc_empty = acc_full + 2;   // [2] epilogue -> MMA
  uint64_t* part_ready = acc_empty + 2;             // [4] per epilogue warp: every block's partials for my tokens are here
  uint64_t* part_free = part_ready + T5_EPI_WARPS;  // [4] per epilogue warp: every owner has read what I stored
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(part_free + T5_EPI_WARPS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_iters = (K + T5_KC - 1) / T5_KC;
  const int rank = csize > 1 ? (int)cluster_rank() : 0;
  const int cluster_id = (int)blockIdx.x / csize, num_clusters = (int)gridDim.x / csize;
  const int my_tiles = cluster_id < num_tiles ? (num_tiles - cluster_id + num_clusters - 1) / num_clusters : 0;
  const int kb0 = rank * kb_per_split;                                   // this block's range of K, in stages
  const int n_kb = min(k_iters, kb0 + kb_per_split) - kb0;

  // producer state (thread 0): stage counter, tile and stage within the tile of the next copy
  long p_it = 0;
  int p_lt = 0, p_kb = 0, ahead = 0;
  int ahead_col[8];
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], T5_EPI_WARPS); }
    for (int q = 0; q < T5_EPI_WARPS; ++q) { mbar_init(&part_ready[q], csize); mbar_init(&part_free[q], csize); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    // W does not depend on the kernel before this one: its first stages are on their way before that kernel ends,
    // and before the rest of this block is set up
    while (ahead < S && p_lt < my_tiles) {
      ahead_col[ahead] = (kb0 + p_kb) * T5_KC;
      mbar_expect_tx(&full[ahead], (unsigned)STAGE_BYTES);
      tma_load_2d(stages + ahead * STAGE_BYTES, &tmW, ahead_col[ahead], (cluster_id + p_lt * num_clusters) * T5_ROWS, &full[ahead]);
      ++ahead; ++p_it;
      if (++p_kb >= n_kb) { p_kb = 0; ++p_lt; }
    }
    tma_prefetch_map(&tmX);
  }
  if (warp == 1) t5_alloc(tmem_slot, TMEM_COLS);   // one warp allocates the tensor memory for the block and publishes its address
  t5_fence_before();
  __syncthreads();
  t5_fence_after();
  if (csize > 1) cluster_sync_all();     // the barriers of every block of the cluster exist before anyone signals them
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------ producer (one thread)
    if (lane == 0) {
      pdl_wait();
      for (int i = 0; i < ahead; ++i)
        tma_load_2d(stages + i * STAGE_BYTES + A_BYTES, &tmX, ahead_col[i], 0, &full[i]);
      for (; p_lt < my_tiles; ++p_it) {
        const int s = (int)(p_it % S);
        if (!mbar_wait(&empty[s], (unsigned)(((p_it / S) - 1) & 1), abort_flag, err)) break;
        const int col = (kb0 + p_kb) * T5_KC;
        mbar_expect_tx(&full[s], (unsigned)STAGE_BYTES);
        tma_load_2d(stages + s * STAGE_BYTES, &tmW, col, (cluster_id + p_lt * num_clusters) * T5_ROWS, &full[s]);
        tma_load_2d(stages + s * STAGE_BYTES + A_BYTES, &tmX, col, 0, &full[s]);
        if (++p_kb >= n_kb) { p_kb = 0; ++p_lt; }
      }
      const long first = p_it > S ? p_it - S : 0;       // copies in flight must land before the block exits
      for (long j = first; j < p_it; ++j) {
        bool done = false;
        for (unsigned i = 0; i < MBAR_SPIN_LIMIT && !done; ++i) done = mbar_try_wait(&full[j % S], (unsigned)((j / S) & 1));
        if (!done) atomicOr(err, VOB_ERR_TIMEOUT_BITS);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer (one thread)
    if (lane == 0) {
      const uint32_t idesc = t5_instr_desc(T5_ROWS, NT);
      long it = 0;
      bool ok = true;
      for (int lt = 0; lt < my_tiles && ok; ++lt) {
        const int a = lt & 1;
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
    const int row = q * 32 + lane;                                // this thread's row of the tile
    // the tokens of a tile are dealt out to the blocks of the cluster: `slice` to each, block r owns [r * slice, ...)
    const int slice = (m_rows + csize - 1) / csize;
    const int my_t0 = rank * slice;
    const int my_tn = max(0, min(m_rows, my_t0 + slice) - my_t0);
    const uint32_t xbuf_addr = smem_addr(xbuf);
    for (int lt = 0; lt < my_tiles; ++lt) {
      const int tile = cluster_id + lt * num_clusters;
      const int a = lt & 1;
      bool ok = mbar_wait(&acc_full[a], (unsigned)((lt >> 1) & 1), abort_flag, err);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      t5_fence_after();
      const long n = (long)tile * T5_ROWS + row;                  // one output feature
      // rows alternate in groups of eight between gate and up: lane l (l & 8 == 0) holds a gate row, lane l + 8 its up row
      const long n_act = (long)tile * (T5_ROWS / 2) + q * 16 + (lane >> 4) * 8 + (lane & 7);
      auto emit = [&](float v, int tok) {                         // the whole warp calls it, for one token
        if (EPI == T5_EPI_SWIGLU) {
          const float up = __shfl_down_sync(0xffffffffu, v, 8);
          if ((lane & 8) == 0 && n_act < N / 2) {
            const float g = t5_round(v);
            const float act = t5_round(g / (1.f + expf(-g)));
            reinterpret_cast<__nv_bfloat16*>(out)[(long)tok * ldo + n_act] = __float2bfloat16_rn(act * t5_round(up));
          }
        } else if (n < N) {
          if (EPI == T5_EPI_F32) reinterpret_cast<float*>(out)[(long)tok * ldo + n] = t5_round(v);
          else reinterpret_cast<__nv_bfloat16*>(out)[(long)tok * ldo + n] = __float2bfloat16_rn(v);
        }
      };
      if (csize == 1) {
#pragma unroll
        for (int c0 = 0; c0 < NT; c0 += 32) {
          if (c0 >= m_rows) break;
          float v[32];
          t5_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * NT + c0), v);
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c0 + j < m_rows) emit(v[j], c0 + j);
        }
        t5_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[a]);
        continue;
      }
      // the owners must have read what this warp stored for the tile before
      if (lt > 0) {
        ok = mbar_wait_cluster(&part_free[q], (unsigned)((lt - 1) & 1), abort_flag, err);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      {
        int owner = 0, tl = 0;
        const uint32_t mine = xbuf_addr + (uint32_t)((rank * slice * T5_ROWS + row) * 4);   // my rows in an owner's buffer
        uint32_t dst = map_to_rank(mine, 0);
#pragma unroll
        for (int c0 = 0; c0 < NT; c0 += 32) {
          if (c0 >= m_rows) break;
          float v[32];
          t5_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * NT + c0), v);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (c0 + j < m_rows) {
              store_remote_f32(dst + (uint32_t)(tl * T5_ROWS * 4), v[j]);
              if (++tl == slice) {
                tl = 0;
                if (++owner < csize) dst = map_to_rank(mine, (uint32_t)owner);
              }
            }
          }
        }
      }
      t5_fence_before();
      asm volatile("fence.acq_rel.cluster;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&acc_empty[a]);
        const uint32_t bar = smem_addr(&part_ready[q]);
        for (int r = 0; r < csize; ++r) mbar_arrive_remote(map_to_rank(bar, (uint32_t)r));
      }
      ok = mbar_wait_cluster(&part_ready[q], (unsigned)(lt & 1), abort_flag, err);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      // this block's tokens: the partials in the order of the K ranges
#pragma unroll 2
      for (int t = 0; t < my_tn; ++t) {
        float s = 0.f;
        for (int r = 0; r < csize; ++r) s += xbuf[((r * slice + t) * T5_ROWS) + row];
        emit(s, my_t0 + t);
      }
      __syncwarp();
      if (lane == 0) {
        const uint32_t bar = smem_addr(&part_free[q]);
        for (int r = 0; r < csize; ++r) mbar_arrive_remote(map_to_rank(bar, (uint32_t)r));
      }
    }
  }
  // every path ends here: the tensor memory goes back before the block exits, and the blocks of a cluster leave
  // together (a block that has gone can no longer be stored to or signalled)
  t5_fence_before();
  __syncthreads();
  if (warp == 1) {
    t5_fence_after();
    t5_dealloc(tmem_base, TMEM_COLS);
  }
  if (csize > 1) cluster_sync_all();
}

static int tc5_sm_count() { return sm_count(); }

// How many clusters of `csize` blocks of this kernel the device runs at once (0 if it cannot run one).
template <int NT, int EPI>
static int tc5_resident_clusters(int csize) {
  static int cached[T5_MAX_CLUSTER + 1] = {0};
  static bool known[T5_MAX_CLUSTER + 1] = {false};
  if (csize < 1 || csize > T5_MAX_CLUSTER) return 0;
  if (known[csize]) return cached[csize];
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc5_kernel<NT, EPI, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, T5Cfg<NT, 1>::SMEM) != cudaSuccess) {
      cudaGetLastError();
      return 0;
    }
    configured = true;
  }
  const int sms = tc5_sm_count();
  int n = 0;
  if (csize == 1) {
    n = sms;
  } else {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(csize * (sms / csize))); cfg.blockDim = dim3(T5_THREADS); cfg.dynamicSmemBytes = T5Cfg<NT, 1>::SMEM;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)csize; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tc5_kernel<NT, EPI, 1>, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
  }
  cached[csize] = n; known[csize] = true;
  return n;
}

// Without clusters a matrix of more tiles than SMs, but fewer than two per SM, runs with two smaller blocks per SM, all
// resident at once: they share the memory bandwidth and end together, where one block per SM would need a second,
// mostly empty round.
static bool tc5_two_per_sm(long tiles, int sms) { return tiles > sms && tiles < 2 * sms; }

// The cluster size for a product [*, K] x [N, K]^T: the one with which the slowest block has the least to read.  A block
// reads `rounds` times its range of K, and a round with a cluster costs an exchange on top; with few blocks at work a
// block cannot read as fast as its share of the memory bandwidth asks, which counts against small grids.
template <int NT, int EPI>
static int tc5_pick_cluster(long N, long K) {
  const long tiles = (N + T5_ROWS - 1) / T5_ROWS, k_iters = (K + T5_KC - 1) / T5_KC;
  const int sms = tc5_sm_count();
  double best_cost = 0.0;
  int best = 1;
  for (int c = 1; c <= T5_MAX_CLUSTER; ++c) {
    const long per = (k_iters + c - 1) / c;
    if (c > 1 && (per * T5_KC < 512 || (c - 1) * per >= k_iters)) continue;
    const long fit = tc5_resident_clusters<NT, EPI>(c);
    if (fit < 1) continue;
    const long clusters = tiles < fit ? tiles : fit, rounds = (tiles + clusters - 1) / clusters;
    const double active = (double)(clusters * c);
    const double slow = active < 120.0 ? 120.0 / active : 1.0;
    double cost = (double)rounds * ((double)per * slow + (c > 1 ? 4.0 : 1.0));
    if (c == 1 && tc5_two_per_sm(tiles, sms)) cost = (double)per * (double)tiles / (double)sms + 1.0;
    if (best_cost == 0.0 || cost < best_cost - 1e-9) { best_cost = cost; best = c; }
  }
  return best;
}

template <int NT, int EPI>
static int tc5_launch(const CUtensorMap* tmW, const CUtensorMap* tmX, void* out, long ldo, int M, int N, int K, int csize,
                      int* err, cudaStream_t stream) {
  if (csize <= 0) csize = tc5_pick_cluster<NT, EPI>(N, K);
  const int num_tiles = (N + T5_ROWS - 1) / T5_ROWS;
  const int k_iters = (K + T5_KC - 1) / T5_KC;
  const int kb_per_split = (k_iters + csize - 1) / csize;
  if ((csize - 1) * kb_per_split >= k_iters) return VOB_BAD_ARGUMENT;      // a K range would be empty
  if (csize == 1 && tc5_two_per_sm(num_tiles, tc5_sm_count())) {
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(gemm_tc5_kernel<NT, EPI, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, T5Cfg<NT, 2>::SMEM);
      if (e != cudaSuccess) return (int)e;
      configured = true;
    }
    return launch_kernel(gemm_tc5_kernel<NT, EPI, 2>, num_tiles, T5_THREADS, T5Cfg<NT, 2>::SMEM, stream, *tmW, *tmX, out, ldo, M, N, K,
                         num_tiles, 1, kb_per_split, err);
  }
  const int fit = tc5_resident_clusters<NT, EPI>(csize);
  if (fit < 1) return VOB_UNSUPPORTED;
  const int clusters = num_tiles < fit ? num_tiles : fit;
  return launch_kernel_cluster(gemm_tc5_kernel<NT, EPI, 1>, clusters * csize, T5_THREADS, T5Cfg<NT, 1>::SMEM, stream, (unsigned)csize,
                               *tmW, *tmX, out, ldo, M, N, K, num_tiles, csize, kb_per_split, err);
}

template <int NT>
static int tc5_dispatch(int epilogue, bool pick_only, const CUtensorMap* tw, const CUtensorMap* tx, void* out, long ldo, int M,
                        int N, int K, int csize, int* err, cudaStream_t stream) {
  if (epilogue == T5_EPI_BF16)
    return pick_only ? tc5_pick_cluster<NT, T5_EPI_BF16>(N, K) : tc5_launch<NT, T5_EPI_BF16>(tw, tx, out, ldo, M, N, K, csize, err, stream);
  if (epilogue == T5_EPI_F32)
    return pick_only ? tc5_pick_cluster<NT, T5_EPI_F32>(N, K) : tc5_launch<NT, T5_EPI_F32>(tw, tx, out, ldo, M, N, K, csize, err, stream);
  if (epilogue == T5_EPI_SWIGLU)
    return pick_only ? tc5_pick_cluster<NT, T5_EPI_SWIGLU>(N, K) : tc5_launch<NT, T5_EPI_SWIGLU>(tw, tx, out, ldo, M, N, K, csize, err, stream);
  return pick_only ? 0 : VOB_BAD_ARGUMENT;
}

}  // namespace vob

using namespace vob;

// Rows of the token box for a step of M tokens (32, 64 or 128).
VOB_API int vob_gemm_tc5_token_box(int M) { return M <= 32 ? 32 : (M <= 64 ? 64 : 128); }

// The cluster size (the number of K ranges) vob_gemm_tc5 chooses for this product on the current device; 0 if none runs.
VOB_API int vob_gemm_tc5_cluster(int M, long N, long K, int epilogue) {
  if (M <= 32) return tc5_dispatch<32>(epilogue, true, nullptr, nullptr, nullptr, 0, M, (int)N, (int)K, 0, nullptr, nullptr);
  if (M <= 64) return tc5_dispatch<64>(epilogue, true, nullptr, nullptr, nullptr, 0, M, (int)N, (int)K, 0, nullptr, nullptr);
  return tc5_dispatch<128>(epilogue, true, nullptr, nullptr, nullptr, 0, M, (int)N, (int)K, 0, nullptr, nullptr);
}

// map_w: vob_tensor_map_bf16_2d of W [N, K] with box rows 128; map_x: of x [M, K] with box rows
// vob_gemm_tc5_token_box(M).  epilogue: 0 bfloat16 out [M,N]; 1 float out [M,N] (rounded to bfloat16 first);
// 2 SiLU(gate)*up over rows that alternate in groups of eight between gate and up, out [M,N/2].  Needs M <= 128.
// cluster: the number of K ranges (blocks of a cluster), 1 to 8; 0 lets the library choose.
VOB_API int vob_gemm_tc5(const void* map_w, const void* map_x, void* out, long ldo, int M, int N, int K, int epilogue,
                         int cluster, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 128 || K <= 0 || K % 8 || !map_w || !map_x || cluster < 0 || cluster > T5_MAX_CLUSTER) return VOB_UNSUPPORTED;
  if (epilogue == T5_EPI_SWIGLU && N % 16) return VOB_BAD_ARGUMENT;
  const CUtensorMap* tw = (const CUtensorMap*)map_w;
  const CUtensorMap* tx = (const CUtensorMap*)map_x;
  if (M <= 32) return tc5_dispatch<32>(epilogue, false, tw, tx, out, ldo, M, N, K, cluster, err, stream);
  if (M <= 64) return tc5_dispatch<64>(epilogue, false, tw, tx, out, ldo, M, N, K, cluster, err, stream);
  return tc5_dispatch<128>(epilogue, false, tw, tx, out, ldo, M, N, K, cluster, err, stream);
}
