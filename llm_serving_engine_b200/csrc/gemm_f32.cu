// True float32 matrix product for the 32-bit path: C[M,N] = A[M,K] * B[N,K]^T (+ bias[N]).
//
// B is a weight matrix kept [out, in] as the checkpoint stores it
// (nn.Linear, reference src/llmserve/model.py:51-66).  Plain FMA on CUDA
// cores: no TF32, no reduced-precision staging.  The k range is cut into at most
// eight ranges of equal length (a multiple of 64, see f32_range); an output
// element is the sum of its ranges' sums in ascending order, starting from zero,
// and a range's sum is one fmaf per k in ascending order, starting from zero.  So
// a row's result does not depend on M, on the tile it falls in, on what else is
// in the batch, or on who adds the ranges up: the kernel itself, or (few rows: a
// block per range, so that enough blocks stream the weights) the kernel that
// consumes the stack of partial sums.
#include "common.cuh"

// Length of a k range: an eighth of K rounded up to a multiple of 64.
__host__ __device__ __forceinline__ int f32_range(int K) { return (((K + 7) / 8 + 63) / 64) * 64; }

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

  float acc[TM][TN], total[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = total[i][j] = 0.f;
  const int range = f32_range(K);   // a multiple of BK

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
    if ((k0 + BK) % range == 0 || k0 + BK >= K) {   // the end of a range: its sum joins the total
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) { total[i][j] += acc[i][j]; acc[i][j] = 0.f; }
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
      float v = total[i][j];
      if (bias) v += bias[n];
      C[(size_t)m * ldc + n] = v;
    }
  }
}

// Few rows (decoding): the job is to stream B once.  A block owns BN = 32 columns and all rows (at most 16);
// thread (column c, row pair g) keeps two sums.  Tiles of 64 k-values of B are read with 16-byte loads that follow
// its rows (coalesced), the next tile is on its way in registers while the current one is worked through, and the
// k-values are added one fmaf at a time in ascending order, range by range: the sums are bit for bit those of the
// kernel above.  gridDim.y == 1: the block adds the ranges up itself.  Else block row y takes range y and writes its
// sum to C + y * part_stride (no bias): the consumer adds the stack up in index order, starting from zero.
// Needs K % 4 == 0 and 16-byte aligned rows of A and B.
constexpr int FEW_BN = 32, FEW_BK = 64, FEW_ROWS = 16, FEW_THREADS = 256;
__global__ void __launch_bounds__(FEW_THREADS)
gemm_f32_few_rows_kernel(const float* __restrict__ A, const float* __restrict__ B, const float* __restrict__ bias,
                         float* __restrict__ C, int M, int N, int K, long long lda, long long ldb, long long ldc,
                         long long part_stride) {
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
  const int range = f32_range(K);
  const bool split = gridDim.y > 1;
  const int k_lo = split ? blockIdx.y * range : 0;
  const int k_hi = split ? min(K, k_lo + range) : K;
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
      b_next[h] = (n < N && k_lo + bk < K) ? *reinterpret_cast<const float4*>(B + (size_t)n * ldb + k_lo + bk) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  pdl_wait();
  a_next = (ar < M && k_lo + ak < K) ? *reinterpret_cast<const float4*>(A + (size_t)ar * lda + k_lo + ak) : make_float4(0.f, 0.f, 0.f, 0.f);
  float acc0 = 0.f, acc1 = 0.f, total0 = 0.f, total1 = 0.f;
  for (int k0 = k_lo; k0 < k_hi; k0 += FEW_BK) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      Bs[bk + 0][br + 16 * h] = b_next[h].x; Bs[bk + 1][br + 16 * h] = b_next[h].y;
      Bs[bk + 2][br + 16 * h] = b_next[h].z; Bs[bk + 3][br + 16 * h] = b_next[h].w;
    }
    As[ak + 0][ar] = a_next.x; As[ak + 1][ar] = a_next.y; As[ak + 2][ar] = a_next.z; As[ak + 3][ar] = a_next.w;
    __syncthreads();
    if (k0 + FEW_BK < k_hi) fetch(k0 + FEW_BK);
#pragma unroll
    for (int kk = 0; kk < FEW_BK; ++kk) {
      const float b = Bs[kk][c];
      acc0 = fmaf(As[kk][2 * g], b, acc0);
      acc1 = fmaf(As[kk][2 * g + 1], b, acc1);
    }
    if ((k0 + FEW_BK) % range == 0 || k0 + FEW_BK >= k_hi) {   // the end of a range
      total0 += acc0; total1 += acc1;
      acc0 = acc1 = 0.f;
    }
    __syncthreads();
  }
  const int n = n0 + c;
  if (n < N) {
    float* dst = C + (split ? (size_t)blockIdx.y * part_stride : 0);
    const float add = (bias && !split) ? bias[n] : 0.f;
    if (2 * g < M) dst[(size_t)(2 * g) * ldc + n] = (bias && !split) ? total0 + add : total0;
    if (2 * g + 1 < M) dst[(size_t)(2 * g + 1) * ldc + n] = (bias && !split) ? total1 + add : total1;
  }
}

// How many ranges the k range of a product is cut into (the height of a stack of partial sums).
extern "C" int lse_gemm_f32_ranges(int K) { return K <= 0 ? 0 : (K + f32_range(K) - 1) / f32_range(K); }

// stack != 0: C is a stack [lse_gemm_f32_ranges(K)][M rows of ldc] (part_stride elements apart) of the ranges' sums,
// for a consumer that adds them up in index order starting from zero; few rows only (M <= 16, K % 4 == 0, aligned),
// no bias.  Whether a product can be had as a stack: lse_gemm_f32_stack_ok.
extern "C" int lse_gemm_f32_stack_ok(const float* A, const float* B, int M, int K, long long lda, long long ldb) {
  return (M > 0 && M <= FEW_ROWS && K > 0 && K % 4 == 0 && lda % 4 == 0 && ldb % 4 == 0 &&
          (((uintptr_t)A | (uintptr_t)B) & 15) == 0) ? 1 : 0;
}

extern "C" int lse_gemm_f32_nt(const float* A, const float* B, const float* bias, float* C, int M,
                               int N, int K, long long lda, long long ldb, long long ldc, int stack,
                               long long part_stride, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return LSE_ERR_BAD_ARGUMENT;
  if (stack) {
    if (!lse_gemm_f32_stack_ok(A, B, M, K, lda, ldb) || bias != nullptr) return LSE_ERR_BAD_ARGUMENT;
    lse_launch(gemm_f32_few_rows_kernel, dim3((N + FEW_BN - 1) / FEW_BN, lse_gemm_f32_ranges(K)), FEW_THREADS, 0, stream,
               A, B, bias, C, M, N, K, lda, ldb, ldc, part_stride);
  } else if (M <= FEW_ROWS && K % 4 == 0 && lda % 4 == 0 && ldb % 4 == 0 && (((uintptr_t)A | (uintptr_t)B) & 15) == 0) {
    lse_launch(gemm_f32_few_rows_kernel, dim3((N + FEW_BN - 1) / FEW_BN), FEW_THREADS, 0, stream, A, B, bias, C, M, N, K,
               lda, ldb, ldc, 0LL);
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
