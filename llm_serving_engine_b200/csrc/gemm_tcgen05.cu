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
//
// GATED_IN: x is not read from memory but made on the way: x[m, k] = silu(gate) * up of the float32
// partial sums gate_up[p][m][k] and gate_up[p][m][inter + k] (the output of the gate/up product,
// K = inter).  Four more warps work the values out (as the SiLU kernel does), write them into the
// stage in the swizzled layout that TMA would leave, and arrive on the stage's barrier beside the
// TMA bytes of w; the same warps read the accumulator back at the end.  Block: 192 threads; at most 16 rows.
template <int BLOCK_N, bool GATED_IN>
__global__ void __launch_bounds__(GATED_IN ? 192 : 128)
gemm_bf16_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                        float* __restrict__ out, int M, int N, int k_tiles, int tiles_per_split, int m_pad,
                        int stages, int kboxes, __nv_bfloat16* __restrict__ gated_out,
                        const float* __restrict__ gate_up, int n_partials, long long partial_stride, int inter,
                        int* __restrict__ arrivals, __nv_bfloat16* __restrict__ finished_out) {
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
      mbar_init(bars + 8u * s, GATED_IN ? 5 : 1);   // the TMA bytes (and the four warps that make x)
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
      const uint32_t tma_bytes = GATED_IN ? (uint32_t)kboxes * A_BYTES : stage_bytes;
      for (int it = 0; it < early; ++it) {
        const uint32_t full = bars + 8u * it;
        mbar_expect_tx(full, tma_bytes);
        for (int b = 0; b < kboxes; ++b)
          tma_load_2d(base + (uint32_t)it * stage_bytes + (uint32_t)b * A_BYTES, &map_w, full,
                      ((tile_lo + it) * kboxes + b) * BLOCK_K, n0);
      }
      pdl_wait();
      LSE_TL_MARK(2)
      for (int it = 0; it < early && !GATED_IN; ++it)
        for (int b = 0; b < kboxes; ++b)
          tma_load_2d(base + (uint32_t)it * stage_bytes + b_base + (uint32_t)b * b_bytes, &map_x, bars + 8u * it,
                      ((tile_lo + it) * kboxes + b) * BLOCK_K, 0);
      for (int it = early; it < n_tiles; ++it) {
        const int s = it % stages;
        const uint32_t parity = (uint32_t)(it / stages) & 1u;
        if (!mbar_wait(bars + 8u * (stages + s), parity ^ 1u, abort_flag)) break;
        const uint32_t full = bars + 8u * s;
        mbar_expect_tx(full, tma_bytes);
        const uint32_t a_dst = base + (uint32_t)s * stage_bytes;
        for (int b = 0; b < kboxes; ++b) {
          const int k = ((tile_lo + it) * kboxes + b) * BLOCK_K;
          tma_load_2d(a_dst + (uint32_t)b * A_BYTES, &map_w, full, k, n0);
          if (!GATED_IN) tma_load_2d(a_dst + b_base + (uint32_t)b * b_bytes, &map_x, full, k, 0);
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

  if (GATED_IN && warp >= 2) {
    // x of every stage: thread -> (row m, 8 consecutive k) = one 16-byte chunk of the row's 128 bytes
    pdl_wait();   // the partial sums come from the kernel before
    const int maker = (int)threadIdx.x - 64;
    unsigned char* stage0 = smem_raw + (base - smem_u32(smem_raw));
    // The partial sums of MAKE_AHEAD stages are fetched together (one round trip to the L2 instead of one
    // per stage).  m_pad is 16 here (the launcher sees to it): 16 rows x 8 chunks = one chunk per thread.
    constexpr int MAKE_AHEAD = 3;
    bool ok = true;
    {
      const int m = maker >> 3, c = maker & 7;
      const float* row = gate_up + (size_t)m * 2 * inter;
      for (int it0 = 0; it0 < n_tiles && ok; it0 += MAKE_AHEAD) {
        float g[MAKE_AHEAD][8], u[MAKE_AHEAD][8];
#pragma unroll
        for (int t = 0; t < MAKE_AHEAD; ++t)
#pragma unroll
          for (int e = 0; e < 8; ++e) g[t][e] = u[t][e] = 0.f;
        for (int p0 = 0; p0 < n_partials; p0 += 2) {   // two partial sums of every stage in flight, added in index order
          float4 v[MAKE_AHEAD][2][4];
#pragma unroll
          for (int t = 0; t < MAKE_AHEAD; ++t) {
            const int k = (tile_lo + it0 + t) * BLOCK_K + c * 8;
            const bool live = it0 + t < n_tiles && m < M && k < inter;   // inter is a multiple of 8: the chunk lies inside the row
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              if (live && p0 + q < n_partials) {
                const float* src = row + (size_t)(p0 + q) * partial_stride + k;
                v[t][q][0] = *reinterpret_cast<const float4*>(src);
                v[t][q][1] = *reinterpret_cast<const float4*>(src + 4);
                v[t][q][2] = *reinterpret_cast<const float4*>(src + inter);
                v[t][q][3] = *reinterpret_cast<const float4*>(src + inter + 4);
              } else {
                v[t][q][0] = v[t][q][1] = v[t][q][2] = v[t][q][3] = make_float4(0.f, 0.f, 0.f, 0.f);
              }
            }
          }
#pragma unroll
          for (int t = 0; t < MAKE_AHEAD; ++t)
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              if (p0 + q < n_partials) {
                g[t][0] += v[t][q][0].x; g[t][1] += v[t][q][0].y; g[t][2] += v[t][q][0].z; g[t][3] += v[t][q][0].w;
                g[t][4] += v[t][q][1].x; g[t][5] += v[t][q][1].y; g[t][6] += v[t][q][1].z; g[t][7] += v[t][q][1].w;
                u[t][0] += v[t][q][2].x; u[t][1] += v[t][q][2].y; u[t][2] += v[t][q][2].z; u[t][3] += v[t][q][2].w;
                u[t][4] += v[t][q][3].x; u[t][5] += v[t][q][3].y; u[t][6] += v[t][q][3].z; u[t][7] += v[t][q][3].w;
              }
            }
        }
#pragma unroll
        for (int t = 0; t < MAKE_AHEAD; ++t) {
          const int it = it0 + t;
          if (it >= n_tiles || !ok) break;
          const int s = it % stages;
          if (it >= stages) {   // one lane waits until the stage is free again and tells the others
            int freed = 1;
            if (lane == 0) freed = mbar_wait(bars + 8u * (stages + s), (((uint32_t)(it / stages)) & 1u) ^ 1u, abort_flag) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, freed, 0) != 0;
          }
          if (!ok) break;
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            // rounded to bfloat16 next: the fast exponential and division are far below that (the SiLU
            // kernel takes the same ones when it writes bfloat16)
            const float a = __fdividef(g[t][2 * e], 1.0f + __expf(-g[t][2 * e])) * u[t][2 * e];
            const float b = __fdividef(g[t][2 * e + 1], 1.0f + __expf(-g[t][2 * e + 1])) * u[t][2 * e + 1];
            const __nv_bfloat162 v2 = __floats2bfloat162_rn(a, b);
            w[e] = *reinterpret_cast<const uint32_t*>(&v2);
          }
          unsigned char* x_tile = stage0 + (size_t)s * stage_bytes + b_base;
          *reinterpret_cast<uint4*>(x_tile + m * 128 + ((c ^ (m & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(bars + 8u * s);   // one arrival per warp
        }
      }
    }
  }

  // epilogue: warp w reads TMEM lanes 32w .. 32w+31 (rows n0 + 32w + lane of w), all m_pad columns
  // (GATED_IN: the four extra warps do, each the quarter of tensor memory that its number gives)
  const int quarter = warp & 3;
  const bool reader = !GATED_IN || warp >= 2;
  pdl_wait();   // nothing is written, and no bounded wait starts, before the earlier kernels are done
  const bool ready = reader && mbar_wait(accum_bar, 0, abort_flag);
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  if (!GATED_IN && ready && gated_out != nullptr) {
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
    const int n = n0 + quarter * ROWS_PER_WARP + lane;
    float* dst = out + (size_t)blockIdx.y * M * N + n;
    for (int c0 = 0; c0 < m_pad; c0 += 8) {
      uint32_t r[8];
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0;
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
  } else if (threadIdx.x == 0 && *abort_flag) {
    // a wait gave up: give copies that may still be in flight time to land before the block leaves
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
  }
  if (!GATED_IN && arrivals != nullptr) {
    // The split of this block column that finishes last (an arrival counter, nobody waits) adds the
    // partial sums of the column's 128 weight rows up in split order: 64 gate rows, then the 64 up
    // rows of the same outputs, and writes silu(gate) * up as bfloat16.  The counter goes back to
    // zero for the next launch.
    __shared__ int last_split;
    __threadfence();
    const int all_ready = __syncthreads_and(ready ? 1 : 0);
    if (threadIdx.x == 0) last_split = all_ready && atomicAdd(&arrivals[blockIdx.x], 1) == (int)gridDim.y - 1;
    __syncthreads();
    if (last_split) {
      __threadfence();
      constexpr int HALF = BLOCK_N / 2;
      const int n_out = N / 2;
      for (int idx = threadIdx.x; idx < M * HALF; idx += 128) {
        const int m = idx / HALF, j = idx % HALF;
        if (n0 + HALF + j >= N) continue;
        float g = 0.f, u = 0.f;
        for (int p = 0; p < (int)gridDim.y; ++p) {
          const float* row = out + ((size_t)p * M + m) * N + n0;
          g += __ldcg(row + j);
          u += __ldcg(row + HALF + j);
        }
        finished_out[(size_t)m * n_out + blockIdx.x * HALF + j] =
            __float2bfloat16_rn(__fdividef(g, 1.0f + __expf(-g)) * u);
      }
      if (threadIdx.x == 0) arrivals[blockIdx.x] = 0;
    }
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

// Queue a copy of the word to `host_dst` (pinned) on `stream`: the host reads it with the step's tokens,
// without a synchronisation of its own.
extern "C" int lse_gemm_bf16_skinny_status_async(int* host_dst, cudaStream_t stream) {
  return (int)cudaMemcpyFromSymbolAsync(host_dst, lse_gemm_error, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
}
extern "C" int lse_gemm_bf16_skinny_status_reset(void) {
  const int zero = 0;
  return (int)cudaMemcpyToSymbol(lse_gemm_error, &zero, sizeof(int));
}

// out[split][m][n] (float32, splits * M * N values) = partial sums of x[M, K] * w[N, K]^T.
// x, w bfloat16 row-major, 16-byte aligned, K a multiple of 8, M <= 256.
namespace {
// GATED_IN: x is null; gate_up[n_partials][M][2 K] float32 (partials `partial_stride` floats apart) gives it.
template <int BLOCK_N, bool GATED_IN = false>
int launch_skinny(const void* x, const void* w, float* out, int M, int N, int K, int splits, int stages, int kboxes,
                  void* gated_out, cudaStream_t stream, const float* gate_up = nullptr, int n_partials = 0,
                  long long partial_stride = 0, int* arrivals = nullptr, void* finished_out = nullptr) {
  if (M <= 0 || N <= 0) return 0;
  const int m_pad = lse_gemm_bf16_skinny_pad(M);
  if (m_pad == 0 || K <= 0 || K % 8 || (((uintptr_t)x | (uintptr_t)w) & 15)) return LSE_ERR_BAD_ARGUMENT;
  if (GATED_IN && (gate_up == nullptr || n_partials < 1 || kboxes != 1 || gated_out != nullptr || m_pad != 16 ||
                   partial_stride % 4 || ((uintptr_t)gate_up & 15)))
    return LSE_ERR_BAD_ARGUMENT;
  if (kboxes != 1 && kboxes != 2 && kboxes != 4) return LSE_ERR_BAD_ARGUMENT;
  if (gated_out != nullptr) {
    if (N % BLOCK_N) return LSE_ERR_BAD_ARGUMENT;
    splits = 1;
  }
  if ((arrivals != nullptr) != (finished_out != nullptr) || (arrivals != nullptr && (N % BLOCK_N || gated_out != nullptr || GATED_IN)))
    return LSE_ERR_BAD_ARGUMENT;
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
  if (!make_map(&map_w, w, N, K, BLOCK_N)) return LSE_ERR_BAD_ARGUMENT;
  if (GATED_IN) map_x = map_w;   // not used
  else if (!make_map(&map_x, x, M, K, m_pad)) return LSE_ERR_BAD_ARGUMENT;
  static size_t configured = 0;   // largest dynamic shared memory asked for so far
  if (smem > configured) {
    cudaError_t err = cudaFuncSetAttribute(gemm_bf16_skinny_kernel<BLOCK_N, GATED_IN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
    configured = smem;
  }
  dim3 grid((N + BLOCK_N - 1) / BLOCK_N, splits);
  cudaError_t err = lse_launch(gemm_bf16_skinny_kernel<BLOCK_N, GATED_IN>, grid, GATED_IN ? 192 : 128, smem, stream,
                               map_w, map_x, out, M, N, k_tiles, per, m_pad, stages, kboxes,
                               (__nv_bfloat16*)gated_out, gate_up, n_partials, partial_stride, K, arrivals,
                               (__nv_bfloat16*)finished_out);
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

// out[split][m][n] = partial sums of x[M, K] * w[N, K]^T where x[m, k] = silu(g) * u (rounded to bfloat16),
// g = sum over p of gate_up[p][m][k], u = sum over p of gate_up[p][m][K + k]: the SiLU gate of the
// feed-forward made inside the product that consumes it.  gate_up: float32, n_partials stacks of [M, 2 K],
// `partial_stride` floats apart, 16-byte aligned; K a multiple of 8; M <= 16 (one chunk of x per thread and stage).
extern "C" int lse_gemm_bf16_skinny_gated_in(const float* gate_up, int n_partials, long long partial_stride,
                                             const void* w, float* out, int M, int N, int K, int splits, int stages,
                                             cudaStream_t stream) {
  return launch_skinny<128, true>(nullptr, w, out, M, N, K, splits, stages, 1, nullptr, stream, gate_up, n_partials,
                                  partial_stride);
}

// The product of lse_gemm_bf16_skinny (128 weight rows per block, any number of splits; `out` gets the
// partial sums as usual) whose last-arriving split of every block column also applies the SiLU gate:
// w holds, per 128 rows, 64 gate rows then the 64 up rows of the same outputs (N a multiple of 128);
// finished_out[M, N / 2] (bfloat16) = silu(sum of gate partials) * (sum of up partials), the sums in
// split order.  `arrivals`: ceil(N / 128) ints that are zero before the first launch (the kernel
// leaves them zero).  One launch at a time may use the same `arrivals`.
extern "C" int lse_gemm_bf16_skinny_finish_gate(const void* x, const void* w, float* out, int* arrivals,
                                                void* finished_out, int M, int N, int K, int splits, int stages,
                                                cudaStream_t stream) {
  if (arrivals == nullptr || finished_out == nullptr) return LSE_ERR_BAD_ARGUMENT;
  return launch_skinny<128>(x, w, out, M, N, K, splits, stages, 1, nullptr, stream, nullptr, 0, 0, arrivals, finished_out);
}
