// bfloat16 matrix product for few rows (decoding): out[m, n] = sum_k x[m, k] * w[n, k]
// on the 5th-generation tensor cores, written to stream the weights at HBM speed.
//
// The product is turned around so that the weights ride the wide side of the
// instruction: one block owns 128 rows of w (the M side of tcgen05.mma, 128 TMEM
// lanes) and all rows of x (the N side, padded to 16/32/.../256 columns).  Tiles
// of 64 k-values are brought in by TMA (128-byte swizzle) through a ring of
// mbarrier-guarded stages; one thread issues the MMAs, the accumulator lives in
// tensor memory, and the four warps read it back with tcgen05.ld.  The k range may
// be split over blockIdx.y; every split writes its own float32 partial sums
// out[split][m][n], and the consumer (norm, rotary, SiLU kernels) adds the partials
// in index order, so results do not depend on timing.
//
// Every wait on an mbarrier is bounded: when it gives up, the block sets
// lse_gemm_error (readable with lse_gemm_bf16_skinny_status), skips its output,
// frees its tensor memory and returns.
#include "tcgen05.cuh"

LSE_TL_DEFINE(lse_timeline_gemm)

namespace {
using namespace tc;
constexpr int BLOCK_K = 64;   // k-values per stage: 128-byte rows
constexpr int UMMA_K = 16;

__device__ int lse_gemm_error;

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  return tc::mbar_wait(bar, parity, abort_flag, &lse_gemm_error);
}
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) { return smem_desc_k_major(addr); }

// BLOCK_N rows of w per block (the M side of the instruction): 128, or 64 for twice as many blocks.
// With 64 the accumulator rows lie in lanes 0-15 of each 32-lane quarter of tensor memory
// (row r -> lane (r % 16) + 32 * (r / 16)).
// grid: (ceil(N / BLOCK_N), splits); block: 128 threads; dynamic shared memory:
// stages * kboxes * (BLOCK_N * 128 B + m_pad * 128 B) + alignment slack + barriers.
template <int BLOCK_N>
__global__ void __launch_bounds__(128)
gemm_bf16_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                        float* __restrict__ out, int M, int N, int k_tiles, int tiles_per_split, int m_pad,
                        int stages, int kboxes, __nv_bfloat16* __restrict__ gated_out) {
  constexpr uint32_t A_BYTES = BLOCK_N * BLOCK_K * 2;
  constexpr int ROWS_PER_WARP = BLOCK_N / 4;   // valid accumulator rows in a warp's quarter of tensor memory
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // a stage holds `kboxes` adjacent 64-wide k-boxes of w, then the same boxes of x: one row of w is
  // then read in pieces of kboxes * 128 contiguous bytes, which DRAM serves better than 128
  const uint32_t b_bytes = (uint32_t)m_pad * BLOCK_K * 2;
  const uint32_t stage_bytes = (uint32_t)kboxes * (A_BYTES + b_bytes);
  const uint32_t b_base = (uint32_t)kboxes * A_BYTES;   // offset of the x boxes inside a stage
  const uint32_t bars = base + (uint32_t)stages * stage_bytes;   // full[stages], empty[stages], accum
  const uint32_t accum_bar = bars + 16u * stages;
  unsigned char* tail = smem_raw + (bars - smem_u32(smem_raw)) + 16 * stages + 8;
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
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 0) {   // one warp allocates the accumulator columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                 ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {   // producer: TMA loads into the ring
      // The weights do not depend on the kernels before this one: their first tiles are
      // fetched at once, while the kernel before may still run.  The rows of x are its
      // output and are fetched after pdl_wait().
      const int early = n_tiles < stages ? n_tiles : stages;
      for (int it = 0; it < early; ++it) {
        const uint32_t full = bars + 8u * it;
        mbar_expect_tx(full, stage_bytes);
        for (int b = 0; b < kboxes; ++b)
          tma_load_2d(base + (uint32_t)it * stage_bytes + (uint32_t)b * A_BYTES, &map_w, full,
                      ((tile_lo + it) * kboxes + b) * BLOCK_K, n0);
      }
      pdl_wait();
      LSE_TL_MARK(2)
      for (int it = 0; it < early; ++it)
        for (int b = 0; b < kboxes; ++b)
          tma_load_2d(base + (uint32_t)it * stage_bytes + b_base + (uint32_t)b * b_bytes, &map_x, bars + 8u * it,
                      ((tile_lo + it) * kboxes + b) * BLOCK_K, 0);
      for (int it = early; it < n_tiles; ++it) {
        const int s = it % stages;
        const uint32_t parity = (uint32_t)(it / stages) & 1u;
        if (!mbar_wait(bars + 8u * (stages + s), parity ^ 1u, abort_flag)) break;
        const uint32_t full = bars + 8u * s;
        mbar_expect_tx(full, stage_bytes);
        const uint32_t a_dst = base + (uint32_t)s * stage_bytes;
        for (int b = 0; b < kboxes; ++b) {
          const int k = ((tile_lo + it) * kboxes + b) * BLOCK_K;
          tma_load_2d(a_dst + (uint32_t)b * A_BYTES, &map_w, full, k, n0);
          tma_load_2d(a_dst + b_base + (uint32_t)b * b_bytes, &map_x, full, k, 0);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {   // MMA issuer
      pdl_wait();      // sleep here, not in a bounded spin, while the kernel before still runs
      // instruction descriptor: D float32, A and B bfloat16, both K-major, N = m_pad, M = 128
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(m_pad >> 3) << 17) |
                             ((uint32_t)(BLOCK_N >> 4) << 24);
      bool ok = true;
      for (int it = 0; it < n_tiles && ok; ++it) {
        const int s = it % stages;
        const uint32_t parity = (uint32_t)(it / stages) & 1u;
        ok = mbar_wait(bars + 8u * s, parity, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t a_src = base + (uint32_t)s * stage_bytes;
        for (int b = 0; b < kboxes; ++b) {
#pragma unroll
          for (int kk = 0; kk < BLOCK_K / UMMA_K; ++kk) {
            const uint64_t da = smem_desc(a_src + (uint32_t)b * A_BYTES + kk * UMMA_K * 2);
            const uint64_t db = smem_desc(a_src + b_base + (uint32_t)b * b_bytes + kk * UMMA_K * 2);
            umma_bf16(tmem_base, da, db, idesc, (it | b | kk) != 0 ? 1u : 0u);
          }
        }
        umma_commit(bars + 8u * (stages + s));   // the stage is free once these MMAs have read it
      }
      if (ok) umma_commit(accum_bar);            // the accumulator is complete
    }
    __syncwarp();
  }

  // epilogue: warp w reads TMEM lanes 32w .. 32w+31 (rows n0 + 32w + lane of w), all m_pad columns
  pdl_wait();   // nothing is written, and no bounded wait starts, before the earlier kernels are done
  const bool ready = mbar_wait(accum_bar, 0, abort_flag);
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  if (ready && gated_out != nullptr) {
    // SiLU gate in the epilogue (one split only): the 128 rows of this block are 64 gate rows, then the
    // 64 up rows of the same outputs.  Warps 2 and 3 hand their (up) values over through shared
    // memory; warps 0 and 1 write silu(gate) * up as bfloat16: gated_out[m][blockIdx.x * 64 + lane].
    float* hand = reinterpret_cast<float*>(smem_raw + (base - smem_u32(smem_raw)));   // stage 0 is free now
    const int pitch = m_pad + 1;
    const int row = (warp & 1) * ROWS_PER_WARP + lane;     // index among the block's BLOCK_N / 2 outputs
    const bool lane_valid = lane < ROWS_PER_WARP;
    float g[8];
    for (int c0 = 0; c0 < m_pad; c0 += 8) {
      uint32_t r[8];
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0;
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                   : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                   : "r"(taddr));
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
      if (warp >= 2 && lane_valid) {
#pragma unroll
        for (int i = 0; i < 8; ++i) hand[row * pitch + c0 + i] = __uint_as_float(r[i]);
      }
      __syncthreads();
      if (warp < 2 && lane_valid) {
        const int col = blockIdx.x * (BLOCK_N / 2) + row;
        if (col < N / 2) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (c0 + i < M) {
              g[i] = __uint_as_float(r[i]);
              const float u = hand[row * pitch + c0 + i];
              gated_out[(size_t)(c0 + i) * (N / 2) + col] = __float2bfloat16_rn((g[i] / (1.0f + expf(-g[i]))) * u);
            }
          }
        }
      }
      __syncthreads();
    }
  } else if (ready) {
    const int n = n0 + warp * ROWS_PER_WARP + lane;
    float* dst = out + (size_t)blockIdx.y * M * N + n;
    for (int c0 = 0; c0 < m_pad; c0 += 8) {
      uint32_t r[8];
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0;
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                   : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                   : "r"(taddr));
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
      if (n < N && lane < ROWS_PER_WARP) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (c0 + i < M) dst[(size_t)(c0 + i) * N] = __uint_as_float(r[i]);
      }
    }
  } else if (threadIdx.x == 0) {
    // a wait gave up: give copies that may still be in flight time to land before the block leaves
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  LSE_TL_MARK(3)
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
}

bool make_map(CUtensorMap* map, const void* ptr, int rows, int cols, int box_rows) {
  return make_map_2d(map, ptr, rows, cols, box_rows);
}
}  // namespace

// Rows of x are padded to this many columns of the instruction (0: more rows than the kernel takes).
extern "C" int lse_gemm_bf16_skinny_pad(int M) {
  for (int pad = 16; pad <= 256; pad *= 2)
    if (M <= pad) return pad;
  return 0;
}

// How many k-splits the launcher will really use for a wish of `splits` (every split gets work).
extern "C" int lse_gemm_bf16_skinny_splits(int K, int splits, int kboxes) {
  if (kboxes != 1 && kboxes != 2 && kboxes != 4) kboxes = 1;
  const int k_tiles = (K + BLOCK_K * kboxes - 1) / (BLOCK_K * kboxes);
  if (splits < 1) splits = 1;
  if (splits > k_tiles) splits = k_tiles;
  const int per = (k_tiles + splits - 1) / splits;
  return (k_tiles + per - 1) / per;
}

// 0: no bounded wait has given up since the library was loaded (synchronises the device).
extern "C" int lse_gemm_bf16_skinny_status(void) {
  int value = 0;
  if (cudaMemcpyFromSymbol(&value, lse_gemm_error, sizeof(int)) != cudaSuccess) return -1;
  return value;
}

// out[split][m][n] (float32, splits * M * N values) = partial sums of x[M, K] * w[N, K]^T.
// x, w bfloat16 row-major, 16-byte aligned, K a multiple of 8, M <= 256.
namespace {
template <int BLOCK_N>
int launch_skinny(const void* x, const void* w, float* out, int M, int N, int K, int splits, int stages, int kboxes,
                  void* gated_out, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  const int m_pad = lse_gemm_bf16_skinny_pad(M);
  if (m_pad == 0 || K <= 0 || K % 8 || (((uintptr_t)x | (uintptr_t)w) & 15)) return LSE_ERR_BAD_ARGUMENT;
  if (kboxes != 1 && kboxes != 2 && kboxes != 4) return LSE_ERR_BAD_ARGUMENT;
  if (gated_out != nullptr) {
    if (N % BLOCK_N) return LSE_ERR_BAD_ARGUMENT;
    splits = 1;
  }
  const int k_tiles = (K + BLOCK_K * kboxes - 1) / (BLOCK_K * kboxes);
  splits = lse_gemm_bf16_skinny_splits(K, splits, kboxes);
  const int per = (k_tiles + splits - 1) / splits;
  const uint32_t stage_bytes = (uint32_t)kboxes * ((uint32_t)BLOCK_N * BLOCK_K * 2 + (uint32_t)m_pad * BLOCK_K * 2);
  if (stages < 2) stages = 2;
  // two blocks must fit on an SM (beside each other, or beside a block of the kernel before): at most
  // about 110 KB of stages per block
  while (stages > 2 && (size_t)stages * stage_bytes + 2048 > 112 * 1024) --stages;
  if (stages > per + 1) stages = per + 1 < 2 ? 2 : per + 1;
  const size_t smem = (size_t)stages * stage_bytes + 1024 + 16 * (size_t)stages + 64;
  CUtensorMap map_w, map_x;
  if (!make_map(&map_w, w, N, K, BLOCK_N) || !make_map(&map_x, x, M, K, m_pad)) return LSE_ERR_BAD_ARGUMENT;
  static size_t configured = 0;   // largest dynamic shared memory asked for so far
  if (smem > configured) {
    cudaError_t err = cudaFuncSetAttribute(gemm_bf16_skinny_kernel<BLOCK_N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
    configured = smem;
  }
  dim3 grid((N + BLOCK_N - 1) / BLOCK_N, splits);
  cudaError_t err = lse_launch(gemm_bf16_skinny_kernel<BLOCK_N>, grid, 128, smem, stream, map_w, map_x, out, M, N,
                               k_tiles, per, m_pad, stages, kboxes, (__nv_bfloat16*)gated_out);
  if (err != cudaSuccess) return (int)err;
  return (int)cudaGetLastError();
}
}  // namespace

// block_n: rows of w per block, 128 or 64.
// gated_out != null: w holds, per block of block_n rows, block_n / 2 gate rows then the block_n / 2 up rows
// of the same outputs; one split is used and gated_out[M, N / 2] (bfloat16) = silu(gate) * up; `out` is
// not written.
extern "C" int lse_gemm_bf16_skinny(const void* x, const void* w, float* out, int M, int N, int K, int splits,
                                    int stages, int kboxes, int block_n, void* gated_out, cudaStream_t stream) {
  if (block_n == 64) return launch_skinny<64>(x, w, out, M, N, K, splits, stages, kboxes, gated_out, stream);
  if (block_n == 128) return launch_skinny<128>(x, w, out, M, N, K, splits, stages, kboxes, gated_out, stream);
  return LSE_ERR_BAD_ARGUMENT;
}
