// Sampling on the device: one block per row of float logits, token id out.
//
// The pipeline is the reference's (vllm-oxide, crates/vllm-oxide/src/sampler.rs:207-261):
// greedy short-circuit (temperature 0 or top_k 1) -> logits * (1/T) -> top-k (ties at the
// threshold are kept, sampler.rs:349-364) -> top-p over the survivors -> Gumbel-max
// argmax(x + g), g = -log(-log(u)).  Argmax ties go to the lowest index (sampler.rs:293-305).
// Two things are this engine's own:
//   * the uniform numbers come from a counter-based generator keyed per row (the caller
//     derives the key from seed, request and step), so a request's tokens do not depend on
//     what shares its batch (the reference draws all rows from one generator, sampler.rs:265-287);
//   * top-p keeps every token whose logit is >= the logit of the boundary token, the first
//     one in descending order at which the cumulative probability reaches p (the reference
//     keeps a prefix of its sort, which is the same set unless equal logits straddle the
//     boundary).  Probability mass is summed as 40-bit fixed point integers, so the set does
//     not depend on the order of summation.
#include "common.cuh"

namespace vob {

constexpr int SAMPLE_THREADS = 1024;
constexpr int SAMPLE_CANDIDATES = 4096;    // tokens that top-p may still keep after one look at the row, held in shared memory

__device__ __forceinline__ uint32_t ordered_key(float x) {
  const uint32_t b = __float_as_uint(x + 0.f);      // -0 becomes +0: equal values get equal keys
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ unsigned long long pack_candidate(float value, int index) {
  return ((unsigned long long)ordered_key(value) << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)index);
}

__device__ __forceinline__ unsigned long long block_max_u64(unsigned long long v, unsigned long long* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
    v = other > v ? other : v;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  unsigned long long r = 0;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) r = scratch[i] > r ? scratch[i] : r;
  return r;
}

// uniform in (0,1), 24 bits, from (row key, token index)
__device__ __forceinline__ float counter_uniform(unsigned long long key, uint32_t index) {
  unsigned long long z = key + ((unsigned long long)index + 1ull) * 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  return ((float)(uint32_t)(z >> 40) + 0.5f) * (1.0f / 16777216.0f);
}

// A histogram update of a whole warp at once: lanes that hit the same bin are found with match.any, their values
// summed with a warp reduction, and one lane per bin adds the sum.  The logits of a row crowd into a few bins (the
// first digit of a key is the sign and most of the exponent), and a 64-bit addition to shared memory is a
// compare-and-swap loop, so this takes top-p from 2.1 ms to 0.5 ms a batch (32-bit counts are quicker left alone).
// Every lane of the warp must call.
// values below 2^41: the low 20 bits and the rest are summed apart (32 lanes of 21 bits fit 32 bits)
__device__ __forceinline__ void warp_hist_mass(unsigned long long* hist, int bin, unsigned long long v, bool active) {
  const unsigned act = __ballot_sync(0xffffffffu, active);
  if (!active) return;
  const unsigned grp = __match_any_sync(act, bin);
  const unsigned lo = __reduce_add_sync(grp, (unsigned)(v & 0xFFFFFull));
  const unsigned hi = __reduce_add_sync(grp, (unsigned)(v >> 20));
  if ((int)(threadIdx.x & 31) == __ffs(grp) - 1) atomicAdd(&hist[bin], ((unsigned long long)hi << 20) + lo);
}

__device__ __forceinline__ unsigned long long fixed_mass(float x, float maxv) {
  return (unsigned long long)(expf(x - maxv) * 1099511627776.0f);  // 2^40
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* logits, long ld, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const unsigned long long* __restrict__ keys, int* __restrict__ out) {
  __shared__ unsigned long long scratch[32];
  __shared__ unsigned int hist[256];
  __shared__ unsigned long long mass[256];
  __shared__ unsigned int s_prefix, s_remaining_k;
  __shared__ unsigned long long s_remaining_mass;
  __shared__ unsigned int s_ncand, s_short, s_gather;
  extern __shared__ unsigned long long cand_raw[];              // SAMPLE_CANDIDATES x (mass, key, index)
  unsigned long long* cand_mass = cand_raw;
  uint32_t* cand_key = reinterpret_cast<uint32_t*>(cand_raw + SAMPLE_CANDIDATES);
  uint32_t* cand_idx = cand_key + SAMPLE_CANDIDATES;
  const int row = blockIdx.x, tid = threadIdx.x;
  const float* l = logits + (size_t)row * ld;
  const float temp = temperature[row];
  const int k = top_k[row];
  const float p = top_p[row];

  if (temp <= 0.f || k == 1) {  // greedy
    unsigned long long best = 0;
    // four logits a load where the row starts on a 16-byte boundary, the rest one by one
    const int v4 = ((uintptr_t)l % 16 == 0) ? V / 4 : 0;
    for (int i = tid; i < v4; i += SAMPLE_THREADS) {
      const float4 x = reinterpret_cast<const float4*>(l)[i];
      const unsigned long long c0 = pack_candidate(x.x, 4 * i), c1 = pack_candidate(x.y, 4 * i + 1);
      const unsigned long long c2 = pack_candidate(x.z, 4 * i + 2), c3 = pack_candidate(x.w, 4 * i + 3);
      const unsigned long long m01 = c0 > c1 ? c0 : c1, m23 = c2 > c3 ? c2 : c3;
      const unsigned long long m = m01 > m23 ? m01 : m23;
      best = m > best ? m : best;
    }
    for (int i = 4 * v4 + tid; i < V; i += SAMPLE_THREADS) {
      const unsigned long long c = pack_candidate(l[i], i);
      best = c > best ? c : best;
    }
    best = block_max_u64(best, scratch);
    if (tid == 0) out[row] = (int)(0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFull));
    return;
  }
  const float inv_t = 1.0f / temp;

  // ---- top-k: key of the k-th largest scaled logit (0 keeps everything)
  // The first digit (sign and most of the exponent) is found over the whole row.  If the tokens whose first digit is
  // at least that of the k-th largest are few, they are gathered into shared memory and everything after (the other
  // three digits, the maximum, top-p, the draw) runs over them alone instead of over the row.
  uint32_t thr = 0;
  bool gathered = false;
  if (k >= 1 && k < V) {
    if (tid == 0) { s_prefix = 0; s_remaining_k = (unsigned)k; s_gather = 0; }
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      if (tid < 256) hist[tid] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const uint32_t mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
      if (gathered) {
        const unsigned ncand = s_ncand;
        for (unsigned c = tid; c < ncand; c += SAMPLE_THREADS) {
          const uint32_t key = cand_key[c];
          if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
      } else {
        for (int i = tid; i < V; i += SAMPLE_THREADS) {
          const uint32_t key = ordered_key(l[i] * inv_t);
          if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
      }
      __syncthreads();
      if (tid == 0) {
        unsigned need = s_remaining_k, cum = 0;
        int b = 255;
        for (; b > 0; --b) {
          if (cum + hist[b] >= need) break;
          cum += hist[b];
        }
        s_remaining_k = need - cum;
        s_prefix = prefix | ((uint32_t)b << shift);
        if (pass == 0 && cum + hist[b] <= (unsigned)SAMPLE_CANDIDATES) { s_gather = 1; s_ncand = 0; }
      }
      __syncthreads();
      if (pass == 0 && s_gather) {
        const uint32_t first = s_prefix >> 24;
        for (int i = tid; i < V; i += SAMPLE_THREADS) {
          const uint32_t key = ordered_key(l[i] * inv_t);
          if ((key >> 24) >= first) {
            const unsigned pos = atomicAdd(&s_ncand, 1u);
            cand_key[pos] = key; cand_idx[pos] = (uint32_t)i;
          }
        }
        gathered = true;
        __syncthreads();
      }
    }
    thr = s_prefix;
  }

  // ---- maximum of the scaled logits (always a survivor)
  unsigned long long best = 0;
  if (gathered) {
    const unsigned ncand = s_ncand;
    for (unsigned c = tid; c < ncand; c += SAMPLE_THREADS) {
      const int i = (int)cand_idx[c];
      const unsigned long long cnd = pack_candidate(l[i] * inv_t, i);
      best = cnd > best ? cnd : best;
    }
  } else {
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
      const unsigned long long c = pack_candidate(l[i] * inv_t, i);
      best = c > best ? c : best;
    }
  }
  best = block_max_u64(best, scratch);
  const int imax = (int)(0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFull));
  const float maxv = l[imax] * inv_t;

  // ---- top-p over the survivors
  if (p > 0.f && p < 1.f) {
    unsigned long long z = 0;
    if (gathered) {
      const unsigned ncand = s_ncand;
      for (unsigned c = tid; c < ncand; c += SAMPLE_THREADS) {
        const unsigned long long m = cand_key[c] >= thr ? fixed_mass(l[cand_idx[c]] * inv_t, maxv) : 0ull;
        cand_mass[c] = m;
        z += m;
      }
    } else {
      for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float x = l[i] * inv_t;
        if (ordered_key(x) >= thr) z += fixed_mass(x, maxv);
      }
    }
    // integer sum over the block: any order gives the same total
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
    __syncthreads();
    if ((tid & 31) == 0) scratch[tid >> 5] = z;
    __syncthreads();
    if (tid == 0) {
      unsigned long long total = 0;
      for (int i = 0; i < SAMPLE_THREADS / 32; ++i) total += scratch[i];
      unsigned long long target = (unsigned long long)((double)p * (double)total);
      if (target < 1) target = 1;
      s_remaining_mass = target;
      s_prefix = 0;
    }
    __syncthreads();
    // The short way.  A token whose mass is below (1 - p) * total / V cannot lie above the boundary unless it IS the
    // boundary token (all tokens after it together weigh less than (1 - p) * total), so the tokens at or above that
    // mass are gathered into shared memory in one pass; if they fit and together reach the target, the boundary is
    // among them and the search (and later the draw) runs over them alone: a language model's distribution leaves
    // a few hundred.  Otherwise (a flat distribution) the row is searched as a whole, four more passes.
    if (tid == 0) { s_short = gathered ? 1u : 0u; if (!gathered) s_ncand = 0; }
    __syncthreads();
    if (!gathered) {
      unsigned long long total = 0;
      for (int i = 0; i < SAMPLE_THREADS / 32; ++i) total += scratch[i];
      const unsigned long long floor_mass = (unsigned long long)((1.0 - (double)p) * (double)total / (double)V);
      if (floor_mass >= 1) {
        for (int i = tid; i < V; i += SAMPLE_THREADS) {
          const float x = l[i] * inv_t;
          const uint32_t key = ordered_key(x);
          if (key < thr) continue;
          const unsigned long long m = fixed_mass(x, maxv);
          if (m < floor_mass) continue;
          const unsigned pos = atomicAdd(&s_ncand, 1u);
          if (pos < (unsigned)SAMPLE_CANDIDATES) { cand_mass[pos] = m; cand_key[pos] = key; cand_idx[pos] = (uint32_t)i; }
        }
      } else if (tid == 0) {
        s_ncand = SAMPLE_CANDIDATES + 1;
      }
    }
    __syncthreads();
    const unsigned ncand = s_ncand;
    if (!gathered && ncand <= (unsigned)SAMPLE_CANDIDATES) {
      unsigned long long z2 = 0;
      for (unsigned i = tid; i < ncand; i += SAMPLE_THREADS) z2 += cand_mass[i];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) z2 += __shfl_xor_sync(0xffffffffu, z2, o);
      __syncthreads();
      if ((tid & 31) == 0) scratch[tid >> 5] = z2;
      __syncthreads();
      if (tid == 0) {
        unsigned long long have = 0;
        for (int i = 0; i < SAMPLE_THREADS / 32; ++i) have += scratch[i];
        s_short = have >= s_remaining_mass ? 1u : 0u;
      }
      __syncthreads();
    }
    const bool short_way = s_short != 0;
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      if (tid < 256) mass[tid] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const uint32_t mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
      if (short_way) {
        for (unsigned i = tid; i < ncand; i += SAMPLE_THREADS) {
          const uint32_t key = cand_key[i];
          if ((key & mask) == prefix) atomicAdd(&mass[(key >> shift) & 255u], cand_mass[i]);
        }
      } else
      for (int base = 0; base < V; base += SAMPLE_THREADS) {
        const int i = base + tid;
        const float x = i < V ? l[i] * inv_t : 0.f;
        const uint32_t key = ordered_key(x);
        const bool in = i < V && key >= thr && (key & mask) == prefix;
        warp_hist_mass(mass, (int)((key >> shift) & 255u), in ? fixed_mass(x, maxv) : 0ull, in);
      }
      __syncthreads();
      if (tid == 0) {
        unsigned long long need = s_remaining_mass, cum = 0;
        int b = 255;
        for (; b > 0; --b) {
          if (cum + mass[b] >= need) break;
          cum += mass[b];
        }
        s_remaining_mass = need - cum;
        s_prefix = prefix | ((uint32_t)b << shift);
      }
      __syncthreads();
    }
    const uint32_t thr_p = s_prefix;
    thr = thr_p > thr ? thr_p : thr;
  }

  // ---- Gumbel-max over the survivors
  const unsigned long long key_row = keys[row];
  best = 0;
  if (gathered || (p > 0.f && p < 1.f && s_short != 0)) {
    // the survivors are among the gathered tokens
    const unsigned ncand = s_ncand;
    for (unsigned c = tid; c < ncand; c += SAMPLE_THREADS) {
      if (cand_key[c] < thr) continue;
      const int i = (int)cand_idx[c];
      const float x = l[i] * inv_t;
      const float u = counter_uniform(key_row, (uint32_t)i);
      const float g = -logf(-logf(u));
      const unsigned long long cnd = pack_candidate(x + g, i);
      best = cnd > best ? cnd : best;
    }
  } else
  for (int i = tid; i < V; i += SAMPLE_THREADS) {
    const float x = l[i] * inv_t;
    if (ordered_key(x) < thr) continue;
    const float u = counter_uniform(key_row, (uint32_t)i);
    const float g = -logf(-logf(u));
    const unsigned long long c = pack_candidate(x + g, i);
    best = c > best ? c : best;
  }
  best = block_max_u64(best, scratch);
  if (tid == 0) out[row] = (int)(0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFull));
}

// Penalties before everything else (sampler.rs:320-345): for each distinct token seen so far,
// logit /= repetition (when != 0), logit -= presence, logit -= frequency * count.
__global__ void penalties_kernel(float* logits, long ld, int V, const int* __restrict__ row_of, const int* __restrict__ token,
                                 const int* __restrict__ count, const float* __restrict__ presence,
                                 const float* __restrict__ frequency, const float* __restrict__ repetition, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int r = row_of[i], tk = token[i];
  if (tk < 0 || tk >= V) return;
  float v = logits[(size_t)r * ld + tk];
  if (repetition[r] != 0.f) v /= repetition[r];
  v -= presence[r];
  if (frequency[r] != 0.f) v -= frequency[r] * (float)count[i];
  logits[(size_t)r * ld + tk] = v;
}

}  // namespace vob

using namespace vob;

VOB_API int vob_sample(const float* logits, long ld, int R, int V, const float* temperature, const int* top_k,
                       const float* top_p, const unsigned long long* keys, int* out, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0) return VOB_BAD_ARGUMENT;
  const int smem = SAMPLE_CANDIDATES * 16;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  sample_kernel<<<R, SAMPLE_THREADS, smem, stream>>>(logits, ld, V, temperature, top_k, top_p, keys, out);
  return launch_status();
}

// (row, token, count) triples: one per distinct token of a row's history; a triple must appear once.
VOB_API int vob_apply_penalties(float* logits, long ld, int V, const int* row_of, const int* token, const int* count,
                                const float* presence, const float* frequency, const float* repetition, int n,
                                cudaStream_t stream) {
  if (n <= 0) return 0;
  penalties_kernel<<<(n + 255) / 256, 256, 0, stream>>>(logits, ld, V, row_of, token, count, presence, frequency,
                                                        repetition, n);
  return launch_status();
}
