// True float32 matrix product C[M,N] = A[M,K] * W[N,K]^T on the CUDA cores (FFMA only: no
// tensor cores, no reduced-precision mode). Every output element is accumulated over k = 0..K-1
// in that order with one fused multiply-add per step, whatever M is and wherever the element
// falls in a tile, so a row's result does not depend on what else is in the batch.
// Stands where the reference's float32 run uses F.linear (miniserve/model/qwen3.py:115-131,186).
#include "common.cuh"

namespace ms {

constexpr int GBM = 64, GBN = 64, GBK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(float* __restrict__ C, const float* __restrict__ A, const float* __restrict__ W, int M, int N, int K,
                int lda, int ldw, int ldc) {
  __shared__ float As[GBK][GBM + 4];
  __shared__ float Ws[GBK][GBN + 4];
  pdl_prologue();
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * GBM, n0 = blockIdx.x * GBN;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, each 4 x 4 outputs
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  // loader mapping: 256 threads, tile 64 x 16 -> each thread 4 elements (one row, 4 consecutive k)
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  for (int k0 = 0; k0 < K; k0 += GBK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      const int am = m0 + lr, wn = n0 + lr;
      As[lk + e][lr] = (am < M && k < K) ? A[(size_t)am * lda + k] : 0.f;
      Ws[lk + e][lr] = (wn < N && k < K) ? W[(size_t)wn * ldw + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GBK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
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
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
    }
  }
}

}  // namespace ms

using namespace ms;

// Padding k beyond K with zeros adds fma(0, 0, acc) = acc exactly, so it does not disturb the order.
MS_EXPORT int ms_gemm_f32(float* C, const float* A, const float* W, int M, int N, int K, int lda, int ldw, int ldc,
                          cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  MS_CHECK_ARG(M > 0 && N > 0 && K > 0, "gemm_f32: bad sizes M=%d N=%d K=%d", M, N, K);
  MS_CHECK_ARG(lda >= K && ldw >= K && ldc >= N, "gemm_f32: leading dimensions too small");
  dim3 grid(ceil_div(N, GBN), ceil_div(M, GBM));
  MS_CHECK_ARG(grid.y <= 65535, "gemm_f32: M=%d too large for one launch", M);
  MS_LAUNCH(gemm_f32_kernel, grid, 256, 0, stream, C, A, W, M, N, K, lda, ldw, ldc);
  return 0;
}
