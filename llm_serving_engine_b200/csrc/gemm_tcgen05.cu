// bfloat16 matrix product for few rows (decoding): out[m, n] = sum_k x[m, k] * w[n, k]
// on the 5th-generation tensor cores, written to stream the weights at HBM speed.
//
// The product is turned around so that the weights ride the wide side of the
// instruction: one block owns BLOCK_N rows of w (the M side of tcgen05.mma, TMEM
// lanes) and all rows of x (the N side, padded to 16/32/.../256 columns).  Tiles
// of 64 k-values are brought in by TMA (128-byte swizzle) through a ring of
// mbarrier-guarded stages; one thread issues the MMAs, the accumulator lives in
// tensor memory, and the four warps read it back with tcgen05.ld.  The k range may
// be split over blockIdx.y; every split writes its own float32 partial sums
// out[split][m][n], and the consumer (norm, rotary, SiLU kernels) adds the partials
// in index order, so results do not depend on timing.  No block waits for another.
//
// Every wait on an mbarrier is bounded: when it gives up, the block sets
// lse_gemm_error (readable with lse_gemm_bf16_skinny_status), skips its output,
// frees its tensor memory and returns.  The limit is lse_gemm_spin_limit (settable, so
// that a test can make a wait run out without waiting long); lse_gemm_test_withhold makes
// the producer leave out its last tile, which is how the test makes a wait run out.
#include "tcgen05.cuh"

LSE_TL_DEFINE(lse_timeline_gemm)

namespace {
using namespace tc;
constexpr int BLOCK_K = 64;   // k-values per stage: 128-byte rows
constexpr int UMMA_K = 16;

__device__ int lse_gemm_error;
__device__ unsigned int lse_gemm_spin_limit = SPIN_LIMIT;
__device__ int lse_gemm_test_withhold;

__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_test_suspend(bar, parity)) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  atomicExch(&lse_gemm_error, 1);
  return false;
}

// BLOCK_N rows of w per block (the M side of the instruction): 128, or 64 for twice as many blocks.
// With 64 the accumulator rows lie in lanes 0-15 of each 32-lane quarter of tensor memory
// (row r -> lane (r % 16) + 32 * (r / 16)).
// grid: (ceil(N / BLOCK_N), splits); block: 128 threads; dynamic shared memory:
// stages * (BLOCK_N * 128 B + m_pad * 128 B) + alignment slack + barriers.
template <int BLOCK_N>
__global__ void __launch_bounds__(128)
gemm_bf16_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                        float* __restrict__ out, int M, int N, int k_tiles, int tiles_per_split, int m_pad, int stages) {
  constexpr uint32_t A_BYTES = BLOCK_N * BLOCK_K * 2;
  constexpr int ROWS_PER_WARP = BLOCK_N / 4;   // valid accumulator rows in a warp's quarter of tensor memory
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t b_bytes = (uint32_t)m_pad * BLOCK_K * 2;
  const uint32_t stage_bytes = A_BYTES + b_bytes;                 // a tile of w, then the same k-values of x
  const uint32_t bars = base + (uint32_t)stages * stage_bytes;   // full[stages], empty[stages], accum
  const uint32_t accum_bar = bars + 16u * stages;
  unsigned char* tail = smem_raw + (accum_bar - smem_u32(smem_raw)) + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BLOCK_N;
  const int tile_lo = blockIdx.y * tiles_per_split;
  const int n_tiles = min(k_tiles, tile_lo + tiles_per_split) - tile_lo;   // >= 1 by the launcher's choice of splits
  const uint32_t tmem_cols = m_pad < 32 ? 32u : (uint32_t)m_pad;

  LSE_TL_BEGIN(5)
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bars + 8u * s, 1);
      mbar_init(bars + 8u * (stages + s), 1);
    }
    mbar_init(accum_bar, 1);
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(tmem_slot, tmem_cols);   // one warp allocates the accumulator columns
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t spin_limit = lse_gemm_spin_limit;
  const int withheld = lse_gemm_test_withhold ? n_tiles - 1 : -1;   // test hook: this tile never arrives

  if (warp == 0) {
    if (lane == 0) {   // producer: TMA loads into the ring
      // The weights do not depend on the kernels before this one: their first tiles are
      // fetched at once, while the kernel before may still run.  The rows of x are its
      // output and are fetched after pdl_wait().
      const int early = n_tiles < stages ? n_tiles : stages;
      for (int it = 0; it < early; ++it) {
        if (it == withheld) continue;
        const uint32_t full = bars + 8u * it;
        mbar_expect_tx(full, stage_bytes);
        tma_load_2d(base + (uint32_t)it * stage_bytes, &map_w, full, (tile_lo + it) * BLOCK_K, n0);
      }
      pdl_wait();
      LSE_TL_MARK(2)
      for (int it = 0; it < early; ++it)
        if (it != withheld)
          tma_load_2d(base + (uint32_t)it * stage_bytes + A_BYTES, &map_x, bars + 8u * it, (tile_lo + it) * BLOCK_K, 0);
      for (int it = early; it < n_tiles; ++it) {
        const int s = it % stages;
        const uint32_t parity = (uint32_t)(it / stages) & 1u;
        if (!wait_bounded(bars + 8u * (stages + s), parity ^ 1u, abort_flag, spin_limit)) break;
        if (it == withheld) continue;
        const uint32_t full = bars + 8u * s;
        mbar_expect_tx(full, stage_bytes);
        const uint32_t dst = base + (uint32_t)s * stage_bytes;
        tma_load_2d(dst, &map_w, full, (tile_lo + it) * BLOCK_K, n0);
        tma_load_2d(dst + A_BYTES, &map_x, full, (tile_lo + it) * BLOCK_K, 0);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {   // MMA issuer
      pdl_wait();      // sleep here, not in a bounded spin, while the kernel before still runs
      // instruction descriptor: D float32, A and B bfloat16, both K-major, N = m_pad, M = BLOCK_N
      const uint32_t idesc = instr_desc_bf16(BLOCK_N, m_pad, false, false);
      bool ok = true;
      for (int it = 0; it < n_tiles && ok; ++it) {
        const int s = it % stages;
        const uint32_t parity = (uint32_t)(it / stages) & 1u;
        ok = wait_bounded(bars + 8u * s, parity, abort_flag, spin_limit);
        if (!ok) break;
        fence_after_sync();
        const uint32_t a_src = base + (uint32_t)s * stage_bytes;
#pragma unroll
        for (int kk = 0; kk < BLOCK_K / UMMA_K; ++kk)
          umma_bf16(tmem_base, smem_desc_k_major(a_src + kk * UMMA_K * 2),
                    smem_desc_k_major(a_src + A_BYTES + kk * UMMA_K * 2), idesc, (it | kk) != 0 ? 1u : 0u);
        umma_commit(bars + 8u * (stages + s));   // the stage is free once these MMAs have read it
      }
      if (ok) umma_commit(accum_bar);            // the accumulator is complete
    }
    __syncwarp();
  }

  // epilogue: warp w reads TMEM lanes 32w .. 32w+31 (rows n0 + w * ROWS_PER_WARP + lane of w), all m_pad columns
  pdl_wait();   // nothing is written, and no bounded wait starts, before the earlier kernels are done
  const bool ready = wait_bounded(accum_bar, 0, abort_flag, spin_limit);
  fence_after_sync();
  LSE_TL_MARK(4)
  if (ready) {
    const int n = n0 + warp * ROWS_PER_WARP + lane;
    float* dst = out + (size_t)blockIdx.y * M * N + n;
    for (int c0 = 0; c0 < m_pad; c0 += 8) {
      uint32_t r[8];
      tmem_ld8(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
      tmem_ld_wait();
      if (n < N && lane < ROWS_PER_WARP) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (c0 + i < M) dst[(size_t)(c0 + i) * N] = __uint_as_float(r[i]);
      }
    }
  } else if (threadIdx.x == 0 && *abort_flag) {
    // a wait gave up: give copies that may still be in flight time to land before the block leaves
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
  }
  fence_before_sync();
  __syncthreads();
  LSE_TL_MARK(3)
  if (warp == 0) tmem_dealloc(tmem_base, tmem_cols);
}
}  // namespace

// Rows of x are padded to this many columns of the instruction (0: more rows than the kernel takes).
extern "C" int lse_gemm_bf16_skinny_pad(int M) {
  for (int pad = 16; pad <= 256; pad *= 2)
    if (M <= pad) return pad;
  return 0;
}

// How many k-splits the launcher will really use for a wish of `splits` (every split gets work).
extern "C" int lse_gemm_bf16_skinny_splits(int K, int splits) {
  const int k_tiles = (K + BLOCK_K - 1) / BLOCK_K;
  if (splits < 1) splits = 1;
  if (splits > k_tiles) splits = k_tiles;
  const int per = (k_tiles + splits - 1) / splits;
  return (k_tiles + per - 1) / per;
}

// 0: no bounded wait has given up since the word was last cleared (synchronises the device).
extern "C" int lse_gemm_bf16_skinny_status(void) {
  int value = 0;
  if (cudaMemcpyFromSymbol(&value, lse_gemm_error, sizeof(int)) != cudaSuccess) return -1;
  return value;
}
// Queue a copy of the word to `host_dst` (pinned) on `stream`: the host reads it with the step's tokens,
// without a synchronisation of its own.
extern "C" int lse_gemm_bf16_skinny_status_async(int* host_dst, cudaStream_t stream) {
  return (int)cudaMemcpyFromSymbolAsync(host_dst, lse_gemm_error, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
}
extern "C" int lse_gemm_bf16_skinny_status_reset(void) {
  const int zero = 0;
  return (int)cudaMemcpyToSymbol(lse_gemm_error, &zero, sizeof(int));
}
// Test hooks.  spin_limit: iterations a bounded wait makes before it gives up (0: the default);
// withhold != 0: every block's producer leaves out its last tile, so that a wait runs out.
extern "C" int lse_gemm_bf16_skinny_test_hooks(unsigned int spin_limit, int withhold) {
  const unsigned int limit = spin_limit ? spin_limit : SPIN_LIMIT;
  cudaError_t err = cudaMemcpyToSymbol(lse_gemm_spin_limit, &limit, sizeof(limit));
  if (err != cudaSuccess) return (int)err;
  return (int)cudaMemcpyToSymbol(lse_gemm_test_withhold, &withhold, sizeof(withhold));
}

namespace {
template <int BLOCK_N>
int launch_skinny(const void* x, const void* w, float* out, int M, int N, int K, int splits, int stages,
                  cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  const int m_pad = lse_gemm_bf16_skinny_pad(M);
  if (m_pad == 0 || K <= 0 || K % 8 || (((uintptr_t)x | (uintptr_t)w) & 15)) return LSE_ERR_BAD_ARGUMENT;
  const int k_tiles = (K + BLOCK_K - 1) / BLOCK_K;
  splits = lse_gemm_bf16_skinny_splits(K, splits);
  const int per = (k_tiles + splits - 1) / splits;
  const uint32_t stage_bytes = (uint32_t)BLOCK_N * BLOCK_K * 2 + (uint32_t)m_pad * BLOCK_K * 2;
  if (stages < 2) stages = 2;
  // two blocks must fit on an SM (beside each other, or beside a block of the kernel before): at most
  // about 110 KB of stages per block
  while (stages > 2 && (size_t)stages * stage_bytes + 2048 > 112 * 1024) --stages;
  if (stages > per + 1) stages = per + 1 < 2 ? 2 : per + 1;
  const size_t smem = (size_t)stages * stage_bytes + 1024 + 16 * (size_t)stages + 64;
  CUtensorMap map_w, map_x;
  if (!make_map_2d(&map_w, w, N, K, BLOCK_N)) return LSE_ERR_BAD_ARGUMENT;
  if (!make_map_2d(&map_x, x, M, K, m_pad)) return LSE_ERR_BAD_ARGUMENT;
  static size_t configured = 0;   // largest dynamic shared memory asked for so far
  if (smem > configured) {
    cudaError_t err = cudaFuncSetAttribute(gemm_bf16_skinny_kernel<BLOCK_N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
    configured = smem;
  }
  dim3 grid((N + BLOCK_N - 1) / BLOCK_N, splits);
  cudaError_t err = lse_launch(gemm_bf16_skinny_kernel<BLOCK_N>, grid, 128, smem, stream, map_w, map_x, out, M, N,
                               k_tiles, per, m_pad, stages);
  if (err != cudaSuccess) return (int)err;
  return (int)cudaGetLastError();
}
}  // namespace

// out[split][m][n] (float32, splits' * M * N values, splits' = lse_gemm_bf16_skinny_splits(K, splits)) =
// partial sums of x[M, K] * w[N, K]^T.  x, w bfloat16 row-major, 16-byte aligned, K a multiple of 8, M <= 256.
// block_n: rows of w per block, 128 or 64.
extern "C" int lse_gemm_bf16_skinny(const void* x, const void* w, float* out, int M, int N, int K, int splits,
                                    int stages, int block_n, cudaStream_t stream) {
  if (block_n == 64) return launch_skinny<64>(x, w, out, M, N, K, splits, stages, stream);
  if (block_n == 128) return launch_skinny<128>(x, w, out, M, N, K, splits, stages, stream);
  return LSE_ERR_BAD_ARGUMENT;
}
