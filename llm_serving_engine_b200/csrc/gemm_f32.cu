// True float32 matrix product for the 32-bit path: C[M,N] = A[M,K] * B[N,K]^T (+ bias[N]).
//
// B is a weight matrix kept [out, in] as the checkpoint stores it
// (nn.Linear, reference src/llmserve/model.py:51-66).  Plain FMA on CUDA
// cores: no TF32, no reduced-precision staging.  Every output element is the
// sum over k = 0..K-1 in that order, one fmaf per k, so a row's result does
// not depend on M, on the tile it falls in or on what else is in the batch.
#include "common.cuh"

template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_f32_nt_kernel(const float* __restrict__ A, const float* __restrict__ B,
                   const float* __restrict__ bias, float* __restrict__ C, int M, int N, int K,
                   long long lda, long long ldb, long long ldc) {
  constexpr int THREADS = (BM / TM) * (BN / TN);
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float As[BK][BM + 1];
  __shared__ float Bs[BK][BN + 1];
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN);  // column group
  const int ty = tid / (BN / TN);  // row group
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // stage A[m0:m0+BM, k0:k0+BK] and B[n0:n0+BN, k0:k0+BK], k fastest in memory
    for (int e = tid; e < BM * BK; e += THREADS) {
      const int r = e / BK, kk = e % BK;
      const int m = m0 + r, k = k0 + kk;
      As[kk][r] = (m < M && k < K) ? A[(size_t)m * lda + k] : 0.f;
    }
    for (int e = tid; e < BN * BK; e += THREADS) {
      const int r = e / BK, kk = e % BK;
      const int n = n0 + r, k = k0 + kk;
      Bs[kk][r] = (n < N && k < K) ? B[(size_t)n * ldb + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
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
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      C[(size_t)m * ldc + n] = v;
    }
  }
}

extern "C" int lse_gemm_f32_nt(const float* A, const float* B, const float* bias, float* C, int M,
                               int N, int K, long long lda, long long ldb, long long ldc,
                               cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return LSE_ERR_BAD_ARGUMENT;
  if (M <= 16) {
    // few rows (decoding): narrow tiles in M so that more blocks stream the weights
    constexpr int BM = 16, BN = 64, BK = 16, TM = 2, TN = 4;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    lse_launch(gemm_f32_nt_kernel<BM, BN, BK, TM, TN>, grid, (BM / TM) * (BN / TN), 0, stream,
               A, B, bias, C, M, N, K, lda, ldb, ldc);
  } else {
    constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    lse_launch(gemm_f32_nt_kernel<BM, BN, BK, TM, TN>, grid, (BM / TM) * (BN / TN), 0, stream,
               A, B, bias, C, M, N, K, lda, ldb, ldc);
  }
  LSE_LAUNCH_CHECK();
}
