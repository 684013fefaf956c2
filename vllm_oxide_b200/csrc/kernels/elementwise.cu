// Row-wise kernels of the forward pass: embedding gather, residual add + RMSNorm,
// bias + per-head RMSNorm + rotation + paged key/value write, SiLU(gate) * up.
//
// Every kernel is a template over the storage type (float for the true 32-bit path,
// bfloat16 for serving).  Sums, norms and rotation are computed in float in both; with
// bfloat16 the values are rounded exactly where the reference rounds them
// (vllm-oxide, crates/vllm-oxide/src/layers/rmsnorm.rs:51-81, layers/rope.rs:129-159,
// layers/activation.rs:17-21).  The order of additions in a row's reduction depends only
// on the row's width, never on what else is in the batch.
#include "common.cuh"

namespace vob {

// ---------------------------------------------------------------- embedding gather
// out[t] = table[ids[t]] * scale (scale 1: a copy; otherwise the product is rounded to T once).
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids, T* __restrict__ out,
                                 int H, int V, float scale, int* err) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int id = ids[t];
  pdl_wait();
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) atomicOr(err, VOB_ERR_TOKEN_ID);
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[(size_t)t * H + i] = from_f<T>(0.f);
    return;
  }
  const T* src = table + (size_t)id * H;
  T* dst = out + (size_t)t * H;
  if (scale != 1.f) {
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = from_f<T>(to_f<T>(src[i]) * scale);
  } else if ((H * sizeof(T)) % 16 == 0) {
    const int4* s4 = reinterpret_cast<const int4*>(src);
    int4* d4 = reinterpret_cast<int4*>(dst);
    const int n = H * sizeof(T) / 16;
    for (int i = threadIdx.x; i < n; i += blockDim.x) d4[i] = s4[i];
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
  }
}

// ---------------------------------------------------------------- residual add + RMSNorm
// One block per output row.  s = x + residual in float; residual' = s rounded to T (written
// in place unless a row list is given); y = round_T(s / sqrt(mean(s^2) + eps)) * w, the
// product rounded to T once more.  With `rows`, output row r is computed from source row
// rows[r] and the residual is left untouched (used for the last norm, on wanted rows only).
template <typename T> struct Vec16;
template <> struct Vec16<float> { static constexpr int N = 4; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T> __device__ __forceinline__ void load16(const T* p, float (&v)[Vec16<T>::N]);
template <> __device__ __forceinline__ void load16<float>(const float* p, float (&v)[4]) {
  const float4 r = *reinterpret_cast<const float4*>(p);
  v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
}
template <> __device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 r = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); v[2 * j] = f.x; v[2 * j + 1] = f.y; }
}
template <typename T> __device__ __forceinline__ void store16(T* p, const float (&v)[Vec16<T>::N]);
template <> __device__ __forceinline__ void store16<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void store16<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 r;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
  *reinterpret_cast<uint4*>(p) = r;
}

template <typename T> __device__ __forceinline__ float2 load2(const T* p);
template <> __device__ __forceinline__ float2 load2<float>(const float* p) { return *reinterpret_cast<const float2*>(p); }
template <> __device__ __forceinline__ float2 load2<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
template <typename T> __device__ __forceinline__ void store2(T* p, float2 v);
template <> __device__ __forceinline__ void store2<float>(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
template <> __device__ __forceinline__ void store2<__nv_bfloat16>(__nv_bfloat16* p, float2 v) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v.x, v.y);
}

// VEC: 16-byte accesses (the row width must be a multiple of 16 bytes); otherwise one element at a time.
// REG > 0: the row's sums stay in registers between the two passes (rows of at most REG * NT 16-byte pieces); else
// they are parked in shared memory.  The order of additions is the same in all three and depends on H only.
template <typename T, int NT, bool VEC, int REG>
__global__ void __launch_bounds__(NT) add_rmsnorm_kernel(const T* x, T* residual, const float* __restrict__ w, T* y,
                                   const int* __restrict__ rows, int H, int num_src_rows, float eps, int has_residual,
                                   int* err) {
  extern __shared__ float srow[];  // H floats (unused with REG)
  __shared__ float scratch[32];
  pdl_launch_dependents();
  const int r = blockIdx.x;
  int src = r;
  pdl_wait();
  if (rows) {
    src = rows[r];
    if (src < 0 || src >= num_src_rows) {
      if (threadIdx.x == 0) atomicOr(err, VOB_ERR_ROW);
      return;
    }
  }
  const T* xr = x + (size_t)src * H;
  T* rr = residual + (size_t)src * H;
  T* yr = y + (size_t)r * H;
  // residual' = x + residual goes back to the residual rows, unless rows were picked, or it is x itself (the norm of a
  // stream that already holds the sum)
  const bool keep = !rows && (has_residual || (const T*)rr != xr);
  float ss = 0.f;
  if (VEC && REG) {
    constexpr int N = Vec16<T>::N, IT = REG > 0 ? REG : 1;
    float v[IT][N];
#pragma unroll
    for (int it = 0; it < IT; ++it) {
      const int i = (threadIdx.x + it * NT) * N;
      if (i < H) {
        load16<T>(xr + i, v[it]);
        if (has_residual) {
          float q[N];
          load16<T>(rr + i, q);
#pragma unroll
          for (int j = 0; j < N; ++j) v[it][j] += q[j];
        }
      }
    }
#pragma unroll
    for (int it = 0; it < IT; ++it) {
      const int i = (threadIdx.x + it * NT) * N;
      if (i < H) {
#pragma unroll
        for (int j = 0; j < N; ++j) ss += v[it][j] * v[it][j];
        if (keep) store16<T>(rr + i, v[it]);
      }
    }
    const float total = block_sum<NT>(ss, scratch);
    const float denom = sqrtf(total / (float)H + eps);
    // 16-bit types: x * (1 / rms) for x / rms, at most one float unit away before the rounding to 16 bits (a float
    // division is ten instructions an element: the kernel was bound by them, 9.1 us for 2,048 rows of 4,096 against
    // 6.2 so); the 32-bit path divides
    const float inv = 1.f / denom;
#pragma unroll
    for (int it = 0; it < IT; ++it) {
      const int i = (threadIdx.x + it * NT) * N;
      if (i < H) {
        float o[N], wv[N];
#pragma unroll
        for (int j = 0; j < N; j += 4) *reinterpret_cast<float4*>(wv + j) = *reinterpret_cast<const float4*>(w + i + j);
#pragma unroll
        for (int j = 0; j < N; ++j) o[j] = round_to<T>(sizeof(T) == 2 ? v[it][j] * inv : v[it][j] / denom) * wv[j];
        store16<T>(yr + i, o);
      }
    }
    return;
  }
  if (VEC) {
    constexpr int N = Vec16<T>::N;
    for (int i = threadIdx.x * N; i < H; i += NT * N) {
      float s[N];
      load16<T>(xr + i, s);
      if (has_residual) {
        float q[N];
        load16<T>(rr + i, q);
#pragma unroll
        for (int j = 0; j < N; ++j) s[j] += q[j];
      }
#pragma unroll
      for (int j = 0; j < N; ++j) { srow[i + j] = s[j]; ss += s[j] * s[j]; }
      if (keep) store16<T>(rr + i, s);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += NT) {
      float s = to_f<T>(xr[i]);
      if (has_residual) s += to_f<T>(rr[i]);
      srow[i] = s;
      ss += s * s;
      if (keep) rr[i] = from_f<T>(s);
    }
  }
  const float total = block_sum<NT>(ss, scratch);
  const float denom = sqrtf(total / (float)H + eps);
  const float inv = 1.f / denom;                  // as above: 16-bit types multiply, the 32-bit path divides
  if (VEC) {
    constexpr int N = Vec16<T>::N;
    for (int i = threadIdx.x * N; i < H; i += NT * N) {
      float o[N];
#pragma unroll
      for (int j = 0; j < N; ++j) o[j] = round_to<T>(sizeof(T) == 2 ? srow[i + j] * inv : srow[i + j] / denom) * w[i + j];
      store16<T>(yr + i, o);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += NT)
      yr[i] = from_f<T>(round_to<T>(sizeof(T) == 2 ? srow[i] * inv : srow[i] / denom) * w[i]);
  }
}

// ---------------------------------------------------------------- SiLU(gate) * up
// gu holds, per token, either I gate values then I up values, or (interleaved) groups of sixteen columns:
// eight gate values and the eight up values of the same outputs.  VEC: eight outputs per thread with 16-byte
// accesses (I a multiple of 8, 16-byte aligned rows).
template <typename T, bool VEC>
__global__ void silu_mul_kernel(const T* gu, T* out, int I, size_t total, int interleaved) {
  pdl_launch_dependents();
  pdl_wait();
  if (VEC) {
    constexpr int N = 8;
    const size_t groups = total / N;
    const int per_row = I / N;
    for (size_t gidx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; gidx < groups; gidx += (size_t)gridDim.x * blockDim.x) {
      // (a 64-bit division is some forty instructions; the groups of nearly every step fit 32 bits)
      const size_t t = groups <= 0xffffffffull ? (size_t)((unsigned)gidx / (unsigned)per_row) : gidx / per_row;
      const int i = (int)(gidx - t * per_row) * N;
      const T* row = gu + t * 2 * I;
      const T* gp = row + (interleaved ? 2 * i : i);
      const T* up = interleaved ? gp + 8 : row + I + i;
      float o[N];
      if (sizeof(T) == 2) {
        float g[8], u[8];
        load16<T>(gp, reinterpret_cast<float(&)[Vec16<T>::N]>(g));
        load16<T>(up, reinterpret_cast<float(&)[Vec16<T>::N]>(u));
#pragma unroll
        for (int j = 0; j < N; ++j) o[j] = round_to<T>(__fdividef(g[j], 1.f + __expf(-g[j]))) * u[j];   // 2 ulp of float: far below bfloat16's step
        store16<T>(out + gidx * N, reinterpret_cast<float(&)[Vec16<T>::N]>(o));
      } else {
#pragma unroll
        for (int j = 0; j < N; ++j) {
          const float g = to_f<T>(gp[j]), u = to_f<T>(up[j]);
          out[gidx * N + j] = from_f<T>(round_to<T>(g / (1.f + expf(-g))) * u);
        }
      }
    }
    return;
  }
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const int gi = interleaved ? (i >> 3) * 16 + (i & 7) : i;
    const int ui = interleaved ? gi + 8 : I + i;
    const float g = to_f<T>(gu[t * 2 * I + gi]);
    const float u = to_f<T>(gu[t * 2 * I + ui]);
    const float s = round_to<T>(g / (1.f + expf(-g)));
    out[idx] = from_f<T>(s * u);
  }
}

// ---------------------------------------------------------------- bias + head norm + rotation + cache write
// A warp takes HPW consecutive heads of one token's merged q|k|v row.  q heads are normalised and rotated in
// place; k heads are normalised, rotated and written to the key cache at the token's slot; v
// heads are copied to the value cache.  cos_sin is [max_pos, hd] float: cos of hd/2 angles, then
// sin.  A slot of -1 writes nothing.  The caches are [pages, kv_heads, block_size, hd]: slot s is row
// s % block_size of page s / block_size, and the rows of one head within a page are contiguous.
// Everything a head needs is a chain of dependent loads, so all loads of all the warp's heads are issued
// before the first is used; with many tokens (prompt portions) a warp takes several heads and shares the
// angles between them.  NV: 64-element steps a lane makes over half a head (hd <= 128 NV).
template <typename T, int NV, int HPW>
__global__ void qk_norm_rope_kv_write_kernel(T* qkv, const T* __restrict__ bias,
                                             const int* __restrict__ positions, const int* __restrict__ slots,
                                             const float* __restrict__ wq, const float* __restrict__ wk,
                                             const float* __restrict__ cos_sin, T* __restrict__ kcache,
                                             T* __restrict__ vcache, int nh, int kvh, int hd, float eps, int max_pos,
                                             long num_slots, int block_size, int write_kv, int* err) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head0 = (blockIdx.y * (blockDim.x >> 5) + warp) * HPW;
  const int total_heads = nh + 2 * kvh;
  const int pos = positions[t];
  const int slot = slots ? slots[t] : -1;
  const int half = hd >> 1;
  const bool pos_ok = pos >= 0 && pos < max_pos;
  // the angles of this token, shared by the warp's heads (they do not depend on the kernel before)
  float2 c[NV], sn[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = 2 * lane + 64 * j;
    if (i < half && pos_ok) {
      c[j] = *reinterpret_cast<const float2*>(cos_sin + (size_t)pos * hd + i);
      sn[j] = *reinterpret_cast<const float2*>(cos_sin + (size_t)pos * hd + i + half);
    }
  }
  pdl_wait();
  if (head0 >= total_heads) return;
  const int width = total_heads * hd;
  // a lane owns pairs (i, i + hd/2) for i = 2*lane, 2*lane+1 (+64, +128, ...): two neighbouring elements per access
  float2 x1[HPW][NV], x2[HPW][NV], wa[HPW][NV], wb[HPW][NV];
#pragma unroll
  for (int h = 0; h < HPW; ++h) {
    const int head = head0 + h;
    if (head >= total_heads) continue;
    const T* row = qkv + (size_t)t * width + (size_t)head * hd;
    const float* w = head < nh ? wq : (head < nh + kvh ? wk : nullptr);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = 2 * lane + 64 * j;
      if (i < half) {
        x1[h][j] = load2<T>(row + i);
        x2[h][j] = load2<T>(row + i + half);
        if (w) {
          wa[h][j] = *reinterpret_cast<const float2*>(w + i);
          wb[h][j] = *reinterpret_cast<const float2*>(w + i + half);
        }
      }
    }
  }
#pragma unroll
  for (int h = 0; h < HPW; ++h) {
    const int head = head0 + h;
    if (head >= total_heads) continue;
    T* row = qkv + (size_t)t * width + (size_t)head * hd;
    const T* brow = bias ? bias + (size_t)head * hd : nullptr;
    const bool is_q = head < nh, is_k = !is_q && head < nh + kvh;
    if (!is_q && (!write_kv || slot < 0)) continue;
    if (!is_q && slot >= num_slots) {
      if (lane == 0) atomicOr(err, VOB_ERR_SLOT);
      continue;
    }
    if (brow) {
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int i = 2 * lane + 64 * j;
        if (i < half) {
          const float2 ba = load2<T>(brow + i), bb = load2<T>(brow + i + half);
          x1[h][j].x = round_to<T>(x1[h][j].x + ba.x); x1[h][j].y = round_to<T>(x1[h][j].y + ba.y);
          x2[h][j].x = round_to<T>(x2[h][j].x + bb.x); x2[h][j].y = round_to<T>(x2[h][j].y + bb.y);
        }
      }
    }
    if (!is_q && !is_k) {  // value head: copy
      T* dst = vcache + (((size_t)(slot / block_size) * kvh + (head - nh - kvh)) * block_size + slot % block_size) * hd;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int i = 2 * lane + 64 * j;
        if (i < half) { store2<T>(dst + i, x1[h][j]); store2<T>(dst + i + half, x2[h][j]); }
      }
      continue;
    }
    if (!pos_ok) {
      if (lane == 0) atomicOr(err, VOB_ERR_POSITION);
      continue;
    }
    if (is_q ? wq != nullptr : wk != nullptr) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < NV; ++j)
        if (2 * lane + 64 * j < half)   // one fixed chain of fused multiply-adds: see the note on the rotation below
          ss = __fmaf_rn(x2[h][j].y, x2[h][j].y, __fmaf_rn(x2[h][j].x, x2[h][j].x,
               __fmaf_rn(x1[h][j].y, x1[h][j].y, __fmaf_rn(x1[h][j].x, x1[h][j].x, ss))));
      ss = warp_sum(ss);
      const float denom = sqrtf(ss / (float)hd + eps);
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        if (2 * lane + 64 * j < half) {
          x1[h][j].x = round_to<T>(round_to<T>(x1[h][j].x / denom) * wa[h][j].x);
          x1[h][j].y = round_to<T>(round_to<T>(x1[h][j].y / denom) * wa[h][j].y);
          x2[h][j].x = round_to<T>(round_to<T>(x2[h][j].x / denom) * wb[h][j].x);
          x2[h][j].y = round_to<T>(round_to<T>(x2[h][j].y / denom) * wb[h][j].y);
        }
      }
    }
    T* dst = is_q ? row : kcache + (((size_t)(slot / block_size) * kvh + (head - nh)) * block_size + slot % block_size) * hd;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = 2 * lane + 64 * j;
      if (i < half) {
        // Products and sums are spelled out (each rounded, none fused): this kernel exists in two shapes (one head or
        // four a warp, chosen by the number of tokens), and left to itself the compiler may fuse a*b - c*d one way in
        // one and another way in the other, which made a token's 32-bit logits depend on the size of its step.
        store2<T>(dst + i, make_float2(__fsub_rn(__fmul_rn(x1[h][j].x, c[j].x), __fmul_rn(x2[h][j].x, sn[j].x)),
                                       __fsub_rn(__fmul_rn(x1[h][j].y, c[j].y), __fmul_rn(x2[h][j].y, sn[j].y))));
        store2<T>(dst + i + half, make_float2(__fadd_rn(__fmul_rn(x2[h][j].x, c[j].x), __fmul_rn(x1[h][j].x, sn[j].x)),
                                              __fadd_rn(__fmul_rn(x2[h][j].y, c[j].y), __fmul_rn(x1[h][j].y, sn[j].y))));
      }
    }
  }
}

// The same for bfloat16 and head sizes 16 * LPH (LPH a power of two up to 32) with 16-byte accesses: LPH lanes share
// a head (a lane owns elements 8*li .. 8*li+7 of both halves), a warp takes 32 / LPH heads.  The quotient
// x / sqrt(..) is formed as x * (1 / sqrt(..)): one float unit of difference at most, far below bfloat16's step.
template <int LPH>
__global__ void qk_norm_rope_kv_write_wide_kernel(__nv_bfloat16* qkv, const __nv_bfloat16* __restrict__ bias,
                                                  const int* __restrict__ positions, const int* __restrict__ slots,
                                                  const float* __restrict__ wq, const float* __restrict__ wk,
                                                  const float* __restrict__ cos_sin, __nv_bfloat16* __restrict__ kcache,
                                                  __nv_bfloat16* __restrict__ vcache, int nh, int kvh, float eps, int max_pos,
                                                  long num_slots, int block_size, int write_kv, int* err) {
  using T = __nv_bfloat16;
  constexpr int HD_ = 16 * LPH, HALF = 8 * LPH, HPW = 32 / LPH;
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int li = lane % LPH;
  const int head = (blockIdx.y * (blockDim.x >> 5) + warp) * HPW + lane / LPH;
  const int total_heads = nh + 2 * kvh;
  const int pos = positions[t];
  const int slot = slots ? slots[t] : -1;
  const bool pos_ok = pos >= 0 && pos < max_pos;
  const int i = li * 8;
  const bool is_q = head < nh, is_k = !is_q && head < nh + kvh, is_v = !is_q && !is_k && head < total_heads;
  const float* w = is_q ? wq : (is_k ? wk : nullptr);
  float c[8], sn[8], wa[8], wb[8];
  if (pos_ok && (is_q || is_k)) {
    const float* cs = cos_sin + (size_t)pos * HD_ + i;
    *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cs);
    *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cs + 4);
    *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(cs + HALF);
    *reinterpret_cast<float4*>(sn + 4) = *reinterpret_cast<const float4*>(cs + HALF + 4);
  }
  if (w) {
    *reinterpret_cast<float4*>(wa) = *reinterpret_cast<const float4*>(w + i);
    *reinterpret_cast<float4*>(wa + 4) = *reinterpret_cast<const float4*>(w + i + 4);
    *reinterpret_cast<float4*>(wb) = *reinterpret_cast<const float4*>(w + HALF + i);
    *reinterpret_cast<float4*>(wb + 4) = *reinterpret_cast<const float4*>(w + HALF + i + 4);
  }
  pdl_wait();
  float x1[8], x2[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) x1[j] = x2[j] = 0.f;
  T* row = qkv + (size_t)t * total_heads * HD_ + (size_t)head * HD_;
  if (head < total_heads) {
    load16<T>(row + i, x1);
    load16<T>(row + i + HALF, x2);
    if (bias) {
      float ba[8], bb[8];
      load16<T>(bias + (size_t)head * HD_ + i, ba);
      load16<T>(bias + (size_t)head * HD_ + i + HALF, bb);
#pragma unroll
      for (int j = 0; j < 8; ++j) { x1[j] = round_to<T>(x1[j] + ba[j]); x2[j] = round_to<T>(x2[j] + bb[j]); }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) ss += x1[j] * x1[j] + x2[j] * x2[j];
#pragma unroll
  for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (head >= total_heads) return;
  if (!is_q) {
    if (!write_kv || slot < 0) return;
    if (slot >= num_slots) {
      if (li == 0) atomicOr(err, VOB_ERR_SLOT);
      return;
    }
  }
  if (is_v) {
    T* dst = vcache + (((size_t)(slot / block_size) * kvh + (head - nh - kvh)) * block_size + slot % block_size) * HD_;
    store16<T>(dst + i, x1);
    store16<T>(dst + i + HALF, x2);
    return;
  }
  if (!pos_ok) {
    if (li == 0) atomicOr(err, VOB_ERR_POSITION);
    return;
  }
  if (w) {
    const float inv = 1.f / sqrtf(ss / (float)HD_ + eps);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      x1[j] = round_to<T>(round_to<T>(x1[j] * inv) * wa[j]);
      x2[j] = round_to<T>(round_to<T>(x2[j] * inv) * wb[j]);
    }
  }
  T* dst = is_q ? row : kcache + (((size_t)(slot / block_size) * kvh + (head - nh)) * block_size + slot % block_size) * HD_;
  float o1[8], o2[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    o1[j] = x1[j] * c[j] - x2[j] * sn[j];
    o2[j] = x2[j] * c[j] + x1[j] * sn[j];
  }
  store16<T>(dst + i, o1);
  store16<T>(dst + i + HALF, o2);
}

// The same for any position rule, one head a warp: the first `rot_dim` elements of a head are rotated (rot_dim even, at
// most hd; 0: no rotation at all), in pairs (i, i + rot_dim/2) or, `interleaved`, in pairs (2i, 2i + 1), by the angle i of
// the token's position; cos_sin is [max_pos, rot_dim]: cos of rot_dim/2 angles, then sin.  The elements from rot_dim on
// pass through (after bias and norm).  The head goes through shared memory, so that a lane finds its partner whatever the
// pairing; the two kernels above are the fast path of the rule "rotate the whole head in halves".
template <typename T>
__global__ void qk_norm_rope_kv_write_general_kernel(T* qkv, const T* __restrict__ bias, const int* __restrict__ positions,
                                                     const int* __restrict__ slots, const float* __restrict__ wq,
                                                     const float* __restrict__ wk, const float* __restrict__ cos_sin,
                                                     T* __restrict__ kcache, T* __restrict__ vcache, int nh, int kvh, int hd,
                                                     int rot_dim, int interleaved, float eps, int max_pos, long num_slots,
                                                     int block_size, int write_kv, int* err) {
  extern __shared__ float head_rows[];   // [warps][hd]
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y * (blockDim.x >> 5) + warp;
  const int total_heads = nh + 2 * kvh;
  const int pos = positions[t];
  const int slot = slots ? slots[t] : -1;
  const bool pos_ok = pos >= 0 && pos < max_pos;
  pdl_wait();
  if (head >= total_heads) return;
  const bool is_q = head < nh, is_k = !is_q && head < nh + kvh;
  if (!is_q && (!write_kv || slot < 0)) return;
  if (!is_q && slot >= num_slots) {
    if (lane == 0) atomicOr(err, VOB_ERR_SLOT);
    return;
  }
  float* x = head_rows + (size_t)warp * hd;
  T* row = qkv + ((size_t)t * total_heads + head) * hd;
  const T* brow = bias ? bias + (size_t)head * hd : nullptr;
  float ss = 0.f;
  for (int d = lane; d < hd; d += 32) {
    float v = to_f<T>(row[d]);
    if (brow) v = round_to<T>(v + to_f<T>(brow[d]));
    x[d] = v;
    ss = __fmaf_rn(v, v, ss);
  }
  if (!is_q && !is_k) {   // value head: copy
    T* dst = vcache + (((size_t)(slot / block_size) * kvh + (head - nh - kvh)) * block_size + slot % block_size) * hd;
    for (int d = lane; d < hd; d += 32) dst[d] = from_f<T>(x[d]);
    return;
  }
  if (rot_dim > 0 && !pos_ok) {
    if (lane == 0) atomicOr(err, VOB_ERR_POSITION);
    return;
  }
  const float* w = is_q ? wq : wk;
  if (w) {
    ss = warp_sum(ss);
    const float denom = sqrtf(ss / (float)hd + eps);
    for (int d = lane; d < hd; d += 32) x[d] = round_to<T>(round_to<T>(x[d] / denom) * w[d]);
  }
  __syncwarp();
  T* dst = is_q ? row : kcache + (((size_t)(slot / block_size) * kvh + (head - nh)) * block_size + slot % block_size) * hd;
  const int half = rot_dim >> 1;
  const float* cs = cos_sin + (size_t)pos * rot_dim;
  for (int d = lane; d < hd; d += 32) {
    float y = x[d];
    if (d < rot_dim) {
      const bool first = interleaved ? !(d & 1) : d < half;
      const int i = interleaved ? d >> 1 : (first ? d : d - half);
      const int partner = interleaved ? d ^ 1 : (first ? d + half : d - half);
      const float c = cs[i], sn = cs[half + i];
      y = first ? __fsub_rn(__fmul_rn(x[d], c), __fmul_rn(x[partner], sn)) : __fadd_rn(__fmul_rn(x[d], c), __fmul_rn(x[partner], sn));
    }
    dst[d] = from_f<T>(y);
  }
}


// ---------------------------------------------------------------- page copy (utility)
template <typename T>
__global__ void copy_pages_kernel(T* cache, const int* __restrict__ pairs, size_t page_elems) {
  const int src = pairs[2 * blockIdx.x], dst = pairs[2 * blockIdx.x + 1];
  for (size_t i = (size_t)blockIdx.y * blockDim.x + threadIdx.x; i < page_elems; i += (size_t)gridDim.y * blockDim.x)
    cache[(size_t)dst * page_elems + i] = cache[(size_t)src * page_elems + i];
}

}  // namespace vob

using namespace vob;

VOB_API int vob_embedding(const void* table, const int* ids, void* out, int T, int H, int V, float scale, int dtype,
                          int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dtype == VOB_F32)
    return launch_kernel(embedding_kernel<float>, T, 128, 0, stream, (const float*)table, ids, (float*)out, H, V, scale, err);
  if (dtype == VOB_BF16)
    return launch_kernel(embedding_kernel<__nv_bfloat16>, T, 128, 0, stream, (const __nv_bfloat16*)table, ids,
                         (__nv_bfloat16*)out, H, V, scale, err);
  return VOB_BAD_ARGUMENT;
}

// logits = cap * tanh(logits / cap), in place, over rows of V floats with row stride ld.
__global__ void softcap_kernel(float* logits, long ld, int V, long total, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  const float inv = 1.f / cap;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    float* p = logits + (i / V) * ld + i % V;
    *p = cap * tanhf(*p * inv);
  }
}

VOB_API int vob_softcap(float* logits, long ld, int R, int V, float cap, cudaStream_t stream) {
  if (R <= 0 || V <= 0) return 0;
  if (!(cap > 0.f)) return VOB_BAD_ARGUMENT;
  const long total = (long)R * V;
  const long want = (total + 255) / 256, most = (long)sm_count() * 16;
  return launch_kernel(softcap_kernel, (int)(want < most ? want : most), 256, 0, stream, logits, ld, V, total, cap);
}

template <typename T>
static int add_rmsnorm_launch(const void* x, void* residual, const float* w, void* y, const int* rows, int n_out, int H,
                              int num_src_rows, float eps, int has_residual, int* err, cudaStream_t stream) {
  constexpr int NT = 256;
  const bool vec = ((size_t)H * sizeof(T)) % 16 == 0 && ((uintptr_t)x | (uintptr_t)residual | (uintptr_t)y) % 16 == 0;
  const int pieces = vec ? (H / Vec16<T>::N + NT - 1) / NT : 0;          // 16-byte pieces of a row per thread
  const int reg = vec && pieces <= 4 && (uintptr_t)w % 16 == 0 ? (pieces <= 1 ? 1 : (pieces <= 2 ? 2 : 4)) : 0;
  const size_t smem = reg ? 0 : (size_t)H * sizeof(float);
  if (smem > 200 * 1024) return VOB_UNSUPPORTED;
  if (smem > 48 * 1024) {
    cudaError_t e = vec ? cudaFuncSetAttribute(add_rmsnorm_kernel<T, NT, true, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                        : cudaFuncSetAttribute(add_rmsnorm_kernel<T, NT, false, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
#define VOB_NORM_LAUNCH(VEC, REG)                                                                                         \
  return launch_kernel(add_rmsnorm_kernel<T, NT, VEC, REG>, n_out, NT, smem, stream, (const T*)x, (T*)residual, w, (T*)y, \
                       rows, H, num_src_rows, eps, has_residual, err)
  if (reg == 1) VOB_NORM_LAUNCH(true, 1);
  if (reg == 2) VOB_NORM_LAUNCH(true, 2);
  if (reg == 4) VOB_NORM_LAUNCH(true, 4);
  if (vec) VOB_NORM_LAUNCH(true, 0);
  VOB_NORM_LAUNCH(false, 0);
#undef VOB_NORM_LAUNCH
}

// y[n_out, H]; x and residual [num_src_rows, H]; rows may be null (then n_out == num_src_rows).
VOB_API int vob_add_rmsnorm(const void* x, void* residual, const float* w, void* y, const int* rows, int n_out, int H,
                            int num_src_rows, float eps, int has_residual, int dtype, int* err, cudaStream_t stream) {
  if (n_out <= 0) return 0;
  if (H <= 0 || (has_residual && !residual)) return VOB_BAD_ARGUMENT;
  if (!has_residual && !rows && !residual) return VOB_BAD_ARGUMENT;  // residual' = x is written there
  if (dtype == VOB_F32) return add_rmsnorm_launch<float>(x, residual, w, y, rows, n_out, H, num_src_rows, eps, has_residual, err, stream);
  if (dtype == VOB_BF16) return add_rmsnorm_launch<__nv_bfloat16>(x, residual, w, y, rows, n_out, H, num_src_rows, eps, has_residual, err, stream);
  return VOB_BAD_ARGUMENT;
}

VOB_API int vob_silu_mul(const void* gu, void* out, int T, int I, int interleaved, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (interleaved && I % 8) return VOB_BAD_ARGUMENT;
  const size_t total = (size_t)T * I;
  const bool vec = I % 8 == 0 && ((uintptr_t)gu | (uintptr_t)out) % 16 == 0;
  const size_t work = vec ? total / 8 : total;
  const size_t cap = (size_t)sm_count() * 16;
  const int blocks = (int)((work + 255) / 256 < cap ? (work + 255) / 256 : cap);
  if (dtype == VOB_F32)
    return vec ? launch_kernel(silu_mul_kernel<float, true>, blocks, 256, 0, stream, (const float*)gu, (float*)out, I, total, interleaved)
               : launch_kernel(silu_mul_kernel<float, false>, blocks, 256, 0, stream, (const float*)gu, (float*)out, I, total, interleaved);
  if (dtype == VOB_BF16)
    return vec ? launch_kernel(silu_mul_kernel<__nv_bfloat16, true>, blocks, 256, 0, stream, (const __nv_bfloat16*)gu,
                               (__nv_bfloat16*)out, I, total, interleaved)
               : launch_kernel(silu_mul_kernel<__nv_bfloat16, false>, blocks, 256, 0, stream, (const __nv_bfloat16*)gu,
                               (__nv_bfloat16*)out, I, total, interleaved);
  return VOB_BAD_ARGUMENT;
}

// The position rule: the first rot_dim elements of every q and k head are rotated (rot_dim even, <= hd; 0: none, cos_sin
// may then be null), in halves or, `interleaved`, in neighbouring pairs; cos_sin is float [max_pos, rot_dim].
VOB_API int vob_qk_norm_rope_kv_write(void* qkv, const void* bias, const int* positions, const int* slots,
                                      const float* wq, const float* wk, const float* cos_sin, void* kcache, void* vcache,
                                      int T, int nh, int kvh, int hd, int rot_dim, int interleaved, float eps, int max_pos,
                                      long num_slots, int block_size, int write_kv, int dtype, int* err,
                                      cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd <= 0 || hd % 2 || hd > 512 || block_size <= 0) return VOB_UNSUPPORTED;
  if ((wq == nullptr) != (wk == nullptr)) return VOB_BAD_ARGUMENT;
  if (rot_dim < 0 || rot_dim > hd || rot_dim % 2 || (rot_dim > 0 && !cos_sin)) return VOB_BAD_ARGUMENT;
  if (rot_dim != hd || interleaved) {
    const int warps = 4;
    dim3 grid(T, (nh + 2 * kvh + warps - 1) / warps);
    const size_t smem = (size_t)warps * hd * sizeof(float);
    if (dtype == VOB_F32)
      return launch_kernel(qk_norm_rope_kv_write_general_kernel<float>, grid, warps * 32, smem, stream, (float*)qkv,
                           (const float*)bias, positions, slots, wq, wk, cos_sin, (float*)kcache, (float*)vcache, nh, kvh, hd,
                           rot_dim, interleaved, eps, max_pos, num_slots, block_size, write_kv, err);
    if (dtype == VOB_BF16)
      return launch_kernel(qk_norm_rope_kv_write_general_kernel<__nv_bfloat16>, grid, warps * 32, smem, stream,
                           (__nv_bfloat16*)qkv, (const __nv_bfloat16*)bias, positions, slots, wq, wk, cos_sin,
                           (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, nh, kvh, hd, rot_dim, interleaved, eps, max_pos,
                           num_slots, block_size, write_kv, err);
    return VOB_BAD_ARGUMENT;
  }
  if (dtype == VOB_BF16 && hd >= 16 && (hd & (hd - 1)) == 0 &&
      (((uintptr_t)qkv | (uintptr_t)bias | (uintptr_t)kcache | (uintptr_t)vcache | (uintptr_t)cos_sin | (uintptr_t)wq | (uintptr_t)wk) % 16) == 0) {
    // head sizes that are a power of two: 16-byte accesses, hd / 16 lanes a head
    const int lph = hd / 16, warps = 4;
    dim3 grid(T, (nh + 2 * kvh + warps * (32 / lph) - 1) / (warps * (32 / lph)));
#define VOB_ROPE_WIDE(LPH)                                                                                                  \
  if (lph == LPH)                                                                                                           \
    return launch_kernel(qk_norm_rope_kv_write_wide_kernel<LPH>, grid, warps * 32, 0, stream, (__nv_bfloat16*)qkv,          \
                         (const __nv_bfloat16*)bias, positions, slots, wq, wk, cos_sin, (__nv_bfloat16*)kcache,             \
                         (__nv_bfloat16*)vcache, nh, kvh, eps, max_pos, num_slots, block_size, write_kv, err)
    VOB_ROPE_WIDE(1); VOB_ROPE_WIDE(2); VOB_ROPE_WIDE(4); VOB_ROPE_WIDE(8); VOB_ROPE_WIDE(16); VOB_ROPE_WIDE(32);
#undef VOB_ROPE_WIDE
  }
  // a warp takes one head when there are few tokens (decoding), four when there are many
  const int nv = hd <= 128 ? 1 : (hd <= 256 ? 2 : 4);
  const int hpw = T >= 256 ? 4 : 1;
  const int warps = 4;
  dim3 grid(T, (nh + 2 * kvh + warps * hpw - 1) / (warps * hpw));
#define VOB_ROPE_LAUNCH(TYPE, NV, HPW)                                                                                   \
  return launch_kernel(qk_norm_rope_kv_write_kernel<TYPE, NV, HPW>, grid, warps * 32, 0, stream, (TYPE*)qkv,            \
                       (const TYPE*)bias, positions, slots, wq, wk, cos_sin, (TYPE*)kcache, (TYPE*)vcache, nh, kvh, hd,  \
                       eps, max_pos, num_slots, block_size, write_kv, err)
#define VOB_ROPE_DISPATCH(TYPE)                                      \
  if (hpw == 1) {                                                    \
    if (nv == 1) VOB_ROPE_LAUNCH(TYPE, 1, 1);                        \
    if (nv == 2) VOB_ROPE_LAUNCH(TYPE, 2, 1);                        \
    VOB_ROPE_LAUNCH(TYPE, 4, 1);                                     \
  }                                                                  \
  if (nv == 1) VOB_ROPE_LAUNCH(TYPE, 1, 4);                          \
  if (nv == 2) VOB_ROPE_LAUNCH(TYPE, 2, 4);                          \
  VOB_ROPE_LAUNCH(TYPE, 4, 4)
  if (dtype == VOB_F32) { VOB_ROPE_DISPATCH(float); }
  if (dtype == VOB_BF16) { VOB_ROPE_DISPATCH(__nv_bfloat16); }
#undef VOB_ROPE_DISPATCH
#undef VOB_ROPE_LAUNCH
  return VOB_BAD_ARGUMENT;
}

// pairs: [n_pairs][2] = (source page, destination page); one cache plane of page_elems elements per page.
VOB_API int vob_copy_pages(void* cache, const int* pairs, int n_pairs, long page_elems, int dtype, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  dim3 grid(n_pairs, 8);
  if (dtype == VOB_F32)
    copy_pages_kernel<float><<<grid, 256, 0, stream>>>((float*)cache, pairs, (size_t)page_elems);
  else if (dtype == VOB_BF16)
    copy_pages_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((__nv_bfloat16*)cache, pairs, (size_t)page_elems);
  else
    return VOB_BAD_ARGUMENT;
  return launch_status();
}

// Programmatic dependent launch on (default) or off, for every kernel of this library.
VOB_API void vob_set_pdl(int on) { pdl_enabled() = on != 0; }

// The number of SMs of the current device, as the launchers of this library see it.
VOB_API int vob_sm_count() { return sm_count(); }

VOB_API const char* vob_error_string(int code) {
  if (code == VOB_BAD_ARGUMENT) return "bad argument to a vllm_oxide_b200 kernel launcher";
  if (code == VOB_UNSUPPORTED) return "size not supported by this vllm_oxide_b200 kernel";
  return cudaGetErrorString((cudaError_t)code);
}
