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

// Few rows (decoding): the job is to stream B once.  A block owns BN = 32 columns and all rows (at most 16);
// thread (column c, row pair g) keeps two sums.  Tiles of 64 k-values of B are read with 16-byte loads that follow
// its rows (coalesced), the next tile is on its way in registers while the current one is worked through, and the
// k-values are still added one fmaf at a time in ascending order: the sums are bit for bit those of the kernel above.
// Needs K % 4 == 0 and 16-byte aligned rows of A and B.
constexpr int FEW_BN = 32, FEW_BK = 64, FEW_ROWS = 16, FEW_THREADS = 256;
__global__ void __launch_bounds__(FEW_THREADS)
gemm_f32_few_rows_kernel(const float* __restrict__ A, const float* __restrict__ B, const float* __restrict__ bias,
                         float* __restrict__ C, int M, int N, int K, long long lda, long long ldb, long long ldc) {
  pdl_launch_dependents();
  __shared__ float Bs[FEW_BK][FEW_BN + 1];
  __shared__ float As[FEW_BK][FEW_ROWS];
  const int tid = threadIdx.x;
  const int c = tid % FEW_BN, g = tid / FEW_BN;   // column of the block, pair of rows (2g, 2g + 1)
  const int n0 = blockIdx.x * FEW_BN;
  // what this thread fetches of a tile: two 16-byte pieces of B (row br, k-values bk .. bk+3 and +32 rows further on),
  // one of A
  const int br = tid / 16, bk = (tid % 16) * 4;   // 16 pieces per row of 64 k-values; rows br and br + 16
  const int ar = tid / 16, ak = (tid % 16) * 4;   // A: 16 rows x 16 pieces
  float4 b_next[2], a_next;
  auto fetch = [&](int k0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int n = n0 + br + 16 * h, k = k0 + bk;
      b_next[h] = (n < N && k < K) ? *reinterpret_cast<const float4*>(B + (size_t)n * ldb + k) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const int k = k0 + ak;
    a_next = (ar < M && k < K) ? *reinterpret_cast<const float4*>(A + (size_t)ar * lda + k) : make_float4(0.f, 0.f, 0.f, 0.f);
  };
  // the first tile of B does not depend on the kernels before this one; A does
  {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int n = n0 + br + 16 * h;
      b_next[h] = (n < N && bk < K) ? *reinterpret_cast<const float4*>(B + (size_t)n * ldb + bk) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  pdl_wait();
  a_next = (ar < M && ak < K) ? *reinterpret_cast<const float4*>(A + (size_t)ar * lda + ak) : make_float4(0.f, 0.f, 0.f, 0.f);
  float acc0 = 0.f, acc1 = 0.f;
  for (int k0 = 0; k0 < K; k0 += FEW_BK) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      Bs[bk + 0][br + 16 * h] = b_next[h].x; Bs[bk + 1][br + 16 * h] = b_next[h].y;
      Bs[bk + 2][br + 16 * h] = b_next[h].z; Bs[bk + 3][br + 16 * h] = b_next[h].w;
    }
    As[ak + 0][ar] = a_next.x; As[ak + 1][ar] = a_next.y; As[ak + 2][ar] = a_next.z; As[ak + 3][ar] = a_next.w;
    __syncthreads();
    if (k0 + FEW_BK < K) fetch(k0 + FEW_BK);
#pragma unroll
    for (int kk = 0; kk < FEW_BK; ++kk) {
      const float b = Bs[kk][c];
      acc0 = fmaf(As[kk][2 * g], b, acc0);
      acc1 = fmaf(As[kk][2 * g + 1], b, acc1);
    }
    __syncthreads();
  }
  const int n = n0 + c;
  if (n < N) {
    const float add = bias ? bias[n] : 0.f;
    if (2 * g < M) C[(size_t)(2 * g) * ldc + n] = bias ? acc0 + add : acc0;
    if (2 * g + 1 < M) C[(size_t)(2 * g + 1) * ldc + n] = bias ? acc1 + add : acc1;
  }
}

extern "C" int lse_gemm_f32_nt(const float* A, const float* B, const float* bias, float* C, int M,
                               int N, int K, long long lda, long long ldb, long long ldc,
                               cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return LSE_ERR_BAD_ARGUMENT;
  if (M <= FEW_ROWS && K % 4 == 0 && lda % 4 == 0 && ldb % 4 == 0 && (((uintptr_t)A | (uintptr_t)B) & 15) == 0) {
    lse_launch(gemm_f32_few_rows_kernel, dim3((N + FEW_BN - 1) / FEW_BN), FEW_THREADS, 0, stream, A, B, bias, C, M, N, K,
               lda, ldb, ldc);
  } else if (M <= 16) {
    // few rows whose width or alignment the kernel above does not take
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
