// Shared helpers of the sm_100a kernels: element types, conversions, reductions, launch checks.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define VOB_API extern "C" __attribute__((visibility("default")))

// dtype codes of the C entry points
#define VOB_F32 0
#define VOB_BF16 1

// bits of the device-side error word (a kernel that meets a bad index skips the access and sets a bit)
#define VOB_ERR_TOKEN_ID 1
#define VOB_ERR_POSITION 2
#define VOB_ERR_SLOT 4
#define VOB_ERR_PAGE 8
#define VOB_ERR_ROW 16

// host-side status codes (beyond cudaError values, which are < 1000)
#define VOB_BAD_ARGUMENT 2001
#define VOB_UNSUPPORTED 2002

namespace vob {

template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// x rounded to the storage type and back: identity for float.
template <typename T> __device__ __forceinline__ float round_to(float x) { return to_f<T>(from_f<T>(x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of NT threads (NT a multiple of 32, at most 1024); every thread gets the result.
// The order of additions depends on NT only.
template <int NT>
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 32 floats */) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < NT / 32; ++i) t += scratch[i];
  return t;
}

// ---- programmatic dependent launch -------------------------------------------------------------
// Kernels of the decode chain are launched so that the next kernel may start while the one before it
// is still running: it sets up, reads what no earlier kernel writes (weights, tables, the step's index
// arrays), and only then waits for the earlier kernel to finish (pdl_wait) before it touches
// activations or the cache.  A kernel launched without the attribute sees both calls as no-ops.
// One rule follows for every kernel launched this way.  Data that another kernel of the same step has written
// (activations, partial results, this step's rows of the cache) must not be read through the non-coherent path: such a
// kernel is alive before its predecessor has finished, and a `const T* __restrict__` parameter lets the compiler use
// ld.global.nc, which then may return what was there before the predecessor wrote (seen as stale queries in decode
// attention inside a CUDA graph).  Pointers to such data are declared WITHOUT __restrict__; weights, tables and
// the step's index arrays, which are complete before the step's first kernel starts, may keep it.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

inline bool& pdl_enabled() { static bool on = true; return on; }

template <typename... KArgs, typename... Args>
inline int launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}

// The same with the blocks grouped into thread-block clusters of `cluster_x` along x (grid.x a multiple of it).
template <typename... KArgs, typename... Args>
inline int launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 unsigned cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_x; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}

// The number of SMs of the current device (asked once; launch shapes are derived from it, never from a literal).
inline int sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
      sms = n;
    else
      return 1;
  }
  return sms;
}

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return static_cast<int>(e);
}

}  // namespace vob
