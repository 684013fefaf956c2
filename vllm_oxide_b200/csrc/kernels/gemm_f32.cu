// C[M,N] = A[M,K] * W[N,K]^T in true 32-bit floats: the matrix product of the 32-bit path.
//
// No tensor cores, no TF32, no split of the K loop: every output element is one chain of
// fused multiply-adds over k = 0..K-1 in ascending order, so its value does not depend on M,
// on the tile it falls into or on what else is in the batch.  64x64 tiles, 16-wide K slices,
// 256 threads with a 4x4 micro-tile each.  Any M, N, K >= 1.
#include "common.cuh"

namespace vob {

constexpr int GM = 64, GN = 64, GK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* A, long lda, const float* __restrict__ W, long ldw, float* C,
                long ldc, const float* __restrict__ bias, int M, int N, int K) {
  __shared__ float As[GK][GM + 4];
  __shared__ float Ws[GK][GN + 4];
  pdl_launch_dependents();
  pdl_wait();
  const int m0 = blockIdx.y * GM, n0 = blockIdx.x * GN;
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;  // micro-tile: rows ty*4.., cols tx*4..
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  // each thread loads 4 elements of A and 4 of W per slice: row = tid / 4, k = (tid % 4) * 4 .. +3
  const int lr = tid / 4, lk = (tid % 4) * 4;
  for (int k0 = 0; k0 < K; k0 += GK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      const int am = m0 + lr, wn = n0 + lr;
      As[lk + j][lr] = (am < M && k < K) ? A[(size_t)am * lda + k] : 0.f;
      Ws[lk + j][lr] = (wn < N && k < K) ? W[(size_t)wn * ldw + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GK; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j] + (bias ? bias[n] : 0.f);
    }
  }
}

}  // namespace vob

using namespace vob;

VOB_API int vob_gemm_f32(const float* A, long lda, const float* W, long ldw, float* C, long ldc, const float* bias,
                         int M, int N, int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return VOB_BAD_ARGUMENT;
  dim3 grid((N + GN - 1) / GN, (M + GM - 1) / GM);
  if (grid.y > 65535) return VOB_UNSUPPORTED;
  return launch_kernel(gemm_f32_kernel, grid, 256, 0, stream, A, lda, W, ldw, C, ldc, bias, M, N, K);
}
