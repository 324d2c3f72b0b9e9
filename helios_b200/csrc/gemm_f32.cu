// True float32 matrix product on the FMA pipes: C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]).
// No tensor cores and no reduced-precision mode.  Every output element is the sum
// over k = 0..K-1 in that order, in one thread, whatever M is: a row's result does
// not depend on the other rows of the launch.   (python/helios/exec/model.py:236-238,
// 250-251, 336-337, 493-496: y = x W^T + b with W stored [out, in].)
#include "common.cuh"

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(float* __restrict__ C, const float* __restrict__ A, const float* __restrict__ W,
                const float* __restrict__ bias, int M, int N, int K, int lda, int ldw, int ldc) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, each TM x TN outputs
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  // each thread loads 4 consecutive k of one row of A and one row of W
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      const int am = m0 + lrow, wn = n0 + lrow;
      As[lk + e][lrow] = (am < M && k < K) ? A[(size_t)am * lda + k] : 0.f;
      Ws[lk + e][lrow] = (wn < N && k < K) ? W[(size_t)wn * ldw + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = Ws[k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j] + (bias ? bias[n] : 0.f);
    }
  }
}

HB_EXPORT int hb_gemm_f32(float* C, const float* A, const float* W, const float* bias, int M, int N,
                          int K, int lda, int ldw, int ldc, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return HB_OK;
  if (K <= 0) return HB_BAD_ARGUMENT;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return HB_BAD_ARGUMENT;
  hb_launch(gemm_f32_kernel, dim3(grid), dim3(256), 0, stream, C, A, W, bias, M, N, K, lda, ldw, ldc);
  return hb_check_launch();
}
