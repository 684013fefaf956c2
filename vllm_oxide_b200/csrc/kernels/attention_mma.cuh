// Building blocks of the bfloat16 attention kernels: m16n8k16 tensor-core products on a 16-row
// query tile, ldmatrix loads from padded shared-memory rows, cp.async copies of cache rows, and the
// online softmax in float (base-2 exponentials; scores are pre-multiplied by log2(e)).
//
// The head size is a compile-time constant: the file that includes this header is compiled once
// per head size with -DVOB_HD=<multiple of 16, at most 256>.
#pragma once
#include "tensor_map.cuh"

#ifndef VOB_HD
#define VOB_HD 128
#endif

namespace vob {

constexpr int HD = VOB_HD;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16 up to 256");
constexpr int ROW_BYTES = HD * 2 + 16;  // one key or value row in shared memory, padded against bank conflicts
constexpr int KSTEPS = HD / 16;         // k-steps of a Q.K^T product
constexpr int DTILES = HD / 8;          // 8-wide output tiles of a P.V product
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0: nothing is read, 16 zero bytes are written
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem_row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem_row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}

// d[16x8] += a[16x16] * b[16x8], bfloat16 in, float accumulate
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 2^x by the hardware approximation (2 ulp; -inf gives 0): the softmax needs no more on the bfloat16 path.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// The largest of three (one instruction on this architecture).
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// One warp's state for a 16-row query tile: the thread owns rows g = lane/4 and g+8.
struct WarpSoftmax {
  float m[2] = {-INFINITY, -INFINITY};  // running maximum (base-2 score domain)
  float l[2] = {0.f, 0.f};              // this thread's part of the running sum
  float o[DTILES][4];                   // weighted value sums: o[j] = (row g: d 8j+2t, +1; row g+8: same)
  __device__ __forceinline__ void clear() {
#pragma unroll
    for (int j = 0; j < DTILES; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  }
};

// Scores of the warp's 16 rows against 16 keys whose rows start at `krows` (shared memory):
// s[0] covers keys 0..7, s[1] keys 8..15; thread holds (row g, keys 2t, 2t+1) and (row g+8, same).
__device__ __forceinline__ void qk_16keys(const uint32_t (&q)[KSTEPS][4], const char* krows, int lane, float (&s)[2][4]) {
#pragma unroll
  for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
  const int mi = lane >> 3, r = lane & 7;
  const char* base = krows + ((mi >> 1) * 8 + r) * ROW_BYTES + (mi & 1) * 16;
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    uint32_t b[4];
    ldmatrix_x4(b, base + ks * 32);
    mma_bf16(s[0], q[ks], b[0], b[1]);
    mma_bf16(s[1], q[ks], b[2], b[3]);
  }
}

// Online-softmax update with the 16 scores per row in s (already scaled to base 2; masked = -inf),
// then o += p * V for the 16 values whose rows start at `vrows`.
__device__ __forceinline__ void softmax_pv_16keys(WarpSoftmax& st, float (&s)[2][4], const char* vrows, int lane) {
  float mx[2];
  mx[0] = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
  mx[1] = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
  }
  float corr[2], mnew[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    mnew[h] = fmaxf(st.m[h], mx[h]);
    corr[h] = (st.m[h] == -INFINITY) ? 0.f : fast_exp2(st.m[h] - mnew[h]);
    st.m[h] = mnew[h];
  }
  float p[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    // a row that has seen no key yet (maximum -inf) gets a finite stand-in, so that -inf - -inf never occurs
    const float m0 = mnew[0] == -INFINITY ? 0.f : mnew[0], m1 = mnew[1] == -INFINITY ? 0.f : mnew[1];
    p[i][0] = fast_exp2(s[i][0] - m0);
    p[i][1] = fast_exp2(s[i][1] - m0);
    p[i][2] = fast_exp2(s[i][2] - m1);
    p[i][3] = fast_exp2(s[i][3] - m1);
  }
  st.l[0] = st.l[0] * corr[0] + (p[0][0] + p[0][1] + p[1][0] + p[1][1]);
  st.l[1] = st.l[1] * corr[1] + (p[0][2] + p[0][3] + p[1][2] + p[1][3]);
  uint32_t a[4];
  a[0] = pack_bf16(p[0][0], p[0][1]);
  a[1] = pack_bf16(p[0][2], p[0][3]);
  a[2] = pack_bf16(p[1][0], p[1][1]);
  a[3] = pack_bf16(p[1][2], p[1][3]);
  const int mi = lane >> 3, r = lane & 7;
  const char* base = vrows + ((mi & 1) * 8 + r) * ROW_BYTES + (mi >> 1) * 16;
#pragma unroll
  for (int j = 0; j < DTILES; j += 2) {
    st.o[j][0] *= corr[0]; st.o[j][1] *= corr[0]; st.o[j][2] *= corr[1]; st.o[j][3] *= corr[1];
    st.o[j + 1][0] *= corr[0]; st.o[j + 1][1] *= corr[0]; st.o[j + 1][2] *= corr[1]; st.o[j + 1][3] *= corr[1];
    uint32_t b[4];
    ldmatrix_x4_trans(b, base + j * 16);
    mma_bf16(st.o[j], a, b[0], b[1]);
    mma_bf16(st.o[j + 1], a, b[2], b[3]);
  }
}

// The cache rows of a tile are copied in runs of 16 keys.  The caches are [pages, kv_heads, block_size, HD],
// pages hold a multiple of 16 keys and tiles start at multiples of 16, so a run lies in one page and is ONE
// contiguous piece of memory for a head.  Looking the pages up is a global load with a long latency, so it is
// done one tile ahead of the copies that need it (tile_pages), into registers.
constexpr int RUN_KEYS = 16;
constexpr int PAGE_NONE = -2;      // no key of the run is wanted: nothing is looked up, zeros are written

template <int TILE>
__device__ __forceinline__ void tile_pages(int (&pages)[TILE / RUN_KEYS], const int* __restrict__ table, int block_size,
                                           int tile_start, int begin, int end) {
#pragma unroll
  for (int run = 0; run < TILE / RUN_KEYS; ++run) {
    const int key0 = tile_start + run * RUN_KEYS;
    pages[run] = (key0 < end && key0 + RUN_KEYS > begin) ? table[key0 / block_size] : PAGE_NONE;
  }
}

// Copies TILE cache rows (keys tile_start .. tile_start+TILE-1 of key/value head kh) into shared memory: K rows
// first, V rows after them; `pages` comes from tile_pages for the same tile.  Keys outside [begin, end) are
// zero-filled (a window group has given the pages below its window back).
template <int TILE, int THREADS>
__device__ __forceinline__ void load_kv_tile(char* stage, const __nv_bfloat16* kcache,
                                             const __nv_bfloat16* vcache, const int (&pages)[TILE / RUN_KEYS],
                                             int block_size, int kvh, int kh, int tile_start, int begin, int end,
                                             long num_pages, int* err) {
  constexpr int CHUNKS = HD / 8;                       // 16-byte chunks per row
  constexpr int RUN_CHUNKS = RUN_KEYS * CHUNKS;
  const long head_off = (long)kh * block_size * HD;
  const long page_elems = (long)kvh * block_size * HD;
#pragma unroll
  for (int run = 0; run < TILE / RUN_KEYS; ++run) {
    const int key0 = tile_start + run * RUN_KEYS;
    const int page = pages[run];
    const bool page_ok = page >= 0 && page < num_pages;
    if (!page_ok && page != PAGE_NONE) atomicOr(err, VOB_ERR_PAGE);
    const long base = page_ok ? (long)page * page_elems + head_off + (long)(key0 % block_size) * HD : 0;
    const __nv_bfloat16* ksrc = kcache + base;
    const __nv_bfloat16* vsrc = vcache + base;
    char* kdst = stage + run * RUN_KEYS * ROW_BYTES;
#pragma unroll
    for (int c = threadIdx.x; c < RUN_CHUNKS; c += THREADS) {
      const int row = c / CHUNKS, col = c - row * CHUNKS;
      const int key = key0 + row;
      const bool valid = page_ok && key >= begin && key < end;
      char* dst = kdst + row * ROW_BYTES + col * 16;
      cp_async16(dst, ksrc + (valid ? c * 8 : 0), valid);
      cp_async16(dst + TILE * ROW_BYTES, vsrc + (valid ? c * 8 : 0), valid);
    }
  }
}

// ---- the same two steps over tiles that TMA wrote: 64-column slices of [rows, 128 bytes], 128-byte swizzled
// (slice s of a tile of ROWS keys starts at s * ROWS * 128 bytes; the tile's base is 1024-byte aligned).
template <int ROWS>
__device__ __forceinline__ void qk_16keys_swizzled(const uint32_t (&q)[KSTEPS][4], const char* ktile, int row0, int lane,
                                                   float (&s)[2][4]) {
#pragma unroll
  for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
  const int mi = lane >> 3, r = lane & 7;
  const int row = row0 + (mi >> 1) * 8 + r;
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    uint32_t b[4];
    ldmatrix_x4(b, ktile + (ks >> 2) * ROWS * 128 + swizzled_offset(row, (ks & 3) * 2 + (mi & 1)));
    mma_bf16(s[0], q[ks], b[0], b[1]);
    mma_bf16(s[1], q[ks], b[2], b[3]);
  }
}

template <int ROWS>
__device__ __forceinline__ void softmax_pv_16keys_swizzled(WarpSoftmax& st, float (&s)[2][4], const char* vtile, int row0,
                                                           int lane) {
  float mx[2];
  mx[0] = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
  mx[1] = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
  }
  float corr[2], mnew[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    mnew[h] = fmaxf(st.m[h], mx[h]);
    corr[h] = (st.m[h] == -INFINITY) ? 0.f : fast_exp2(st.m[h] - mnew[h]);
    st.m[h] = mnew[h];
  }
  float p[2][4];
  const float m0 = mnew[0] == -INFINITY ? 0.f : mnew[0], m1 = mnew[1] == -INFINITY ? 0.f : mnew[1];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    p[i][0] = fast_exp2(s[i][0] - m0);
    p[i][1] = fast_exp2(s[i][1] - m0);
    p[i][2] = fast_exp2(s[i][2] - m1);
    p[i][3] = fast_exp2(s[i][3] - m1);
  }
  st.l[0] = st.l[0] * corr[0] + (p[0][0] + p[0][1] + p[1][0] + p[1][1]);
  st.l[1] = st.l[1] * corr[1] + (p[0][2] + p[0][3] + p[1][2] + p[1][3]);
  uint32_t a[4];
  a[0] = pack_bf16(p[0][0], p[0][1]);
  a[1] = pack_bf16(p[0][2], p[0][3]);
  a[2] = pack_bf16(p[1][0], p[1][1]);
  a[3] = pack_bf16(p[1][2], p[1][3]);
  const int mi = lane >> 3, r = lane & 7;
  const int row = row0 + (mi & 1) * 8 + r;
#pragma unroll
  for (int j = 0; j < DTILES; j += 2) {
    st.o[j][0] *= corr[0]; st.o[j][1] *= corr[0]; st.o[j][2] *= corr[1]; st.o[j][3] *= corr[1];
    st.o[j + 1][0] *= corr[0]; st.o[j + 1][1] *= corr[0]; st.o[j + 1][2] *= corr[1]; st.o[j + 1][3] *= corr[1];
    const int d0 = j * 8 + (mi >> 1) * 8;      // first of the eight value columns this lane's row address names
    uint32_t b[4];
    ldmatrix_x4_trans(b, vtile + (d0 >> 6) * ROWS * 128 + swizzled_offset(row, (d0 & 63) >> 3));
    mma_bf16(st.o[j], a, b[0], b[1]);
    mma_bf16(st.o[j + 1], a, b[2], b[3]);
  }
}

// Page ids for a TMA producer warp.  A look-up is a global load with a long latency, and a producer that needs
// one per tile cannot run ahead of it; so the warp's 32 lanes fetch the pages of 32 runs of 16 keys (8 tiles) at
// once, one chunk ahead of their use, and hand them to the issuing lane by shuffle.
struct WarpPages {
  int cur = PAGE_NONE, next = PAGE_NONE;   // this lane's run in the current and in the next chunk
  __device__ __forceinline__ int fetch(const int* __restrict__ table, int block_size, int first_key, int chunk, int lane,
                                       int begin, int end) const {
    const int key0 = first_key + (chunk * 32 + lane) * RUN_KEYS;
    return (key0 < end && key0 + RUN_KEYS > begin) ? table[key0 / block_size] : PAGE_NONE;
  }
  // call with all lanes at tile `it` (tiles of 64 keys = 4 runs) before `page()`
  __device__ __forceinline__ void advance(const int* __restrict__ table, int block_size, int first_key, int it, int lane,
                                          int begin, int end) {
    if ((it & 7) == 0) {
      const int chunk = it >> 3;
      cur = it == 0 ? fetch(table, block_size, first_key, 0, lane, begin, end) : next;
      next = fetch(table, block_size, first_key, chunk + 1, lane, begin, end);
    }
  }
  // page of run `run` (0..3) of tile `it`, the same value in every lane
  __device__ __forceinline__ int page(int it, int run) const { return __shfl_sync(0xffffffffu, cur, ((it & 7) << 2) + run); }
};

}  // namespace vob
