// bfloat16 matrix product for few rows (decoding): y[m, n] = sum_k x[m, k] * w[n, k]
// on the 5th-generation tensor cores, written to stream the weights at HBM speed and to
// take the small kernels around a product into the product itself.
//
// The product is turned around so that the weights ride the wide side of the instruction:
// one block owns BLOCK_N rows of w (the M side of tcgen05.mma, TMEM lanes) and all rows of
// x (the N side, padded to 16 or 32 columns).  Tiles of 64 k-values of w are brought in by
// TMA (128-byte swizzle) through a ring of mbarrier-guarded stages; one thread issues the
// MMAs, the accumulator lives in tensor memory, and the four warps read it back with
// tcgen05.ld.  The k range is cut into `splits` pieces so that enough blocks stream.
//
// Where x comes from (NORM_X):
//   false  x is a bfloat16 matrix in memory; its tiles come by TMA beside those of w.
//   true   x is made on the way: x[m, k] = (r[m, k] * inv[m]) * g[k], the RMSNorm of the float32
//          residual rows r with norm weights g; inv[m] = rsqrt(sum_p sumsq[p][m] / K + eps), where
//          sumsq[p][m] are partial sums of squares of row m that the producer of r left (added in
//          index order).  The block's threads write its k range of x into shared memory in the
//          layout TMA would leave; no norm kernel runs and no normalised rows pass through memory.
//
// What happens to the sums (EPI):
//   PARTIALS  every split writes its own float32 partial sums out[split][m][n]; the consumer adds them
//             in index order.  No block waits for another.
//   the others: the splits of one block column form a thread-block CLUSTER.  Every block leaves its
//   accumulator in its own shared memory; after a cluster barrier block r of the cluster adds up, in
//   split order, its share of the columns from all blocks' shared memory (distributed shared memory)
//   and finishes them:
//   PLAIN     out[m][n] = sum (+ bias[n]), float32.
//   RESIDUAL  r[m][n] += sum (the float32 residual stream, in place), and the sum of squares of the new
//             r[m][n] over the block's share of columns goes to sumsq[column block * splits + rank][m]:
//             the next product's NORM_X reads both.
//   GATE      w holds, per BLOCK_N rows, BLOCK_N / 2 gate rows then the BLOCK_N / 2 up rows of the same
//             outputs: act[m][j] = silu(gate sum) * (up sum) as bfloat16 (the SwiGLU activations).
//   Sums are added in split order whatever finishes first, so results do not depend on timing.
//
// Every wait on an mbarrier is bounded: when it gives up, the block sets lse_gemm_error (readable with
// lse_gemm_bf16_skinny_status), contributes zeros, still takes part in the cluster's barriers (nobody is
// left waiting), frees its tensor memory and returns.  The limit is lse_gemm_spin_limit (settable, so
// that a test can make a wait run out without waiting long); lse_gemm_test_withhold makes the producer
// skip its last tile, which is how the test makes a wait run out.
#include <cooperative_groups.h>

#include "tcgen05.cuh"

namespace cg = cooperative_groups;

LSE_TL_DEFINE(lse_timeline_gemm)

namespace {
using namespace tc;
constexpr int BLOCK_K = 64;   // k-values per stage: 128-byte rows
constexpr int UMMA_K = 16;

enum Epilogue { PARTIALS = 0, PLAIN = 1, RESIDUAL = 2, GATE = 3 };

__device__ int lse_gemm_error;
__device__ unsigned int lse_gemm_spin_limit = SPIN_LIMIT;
__device__ int lse_gemm_test_withhold;

struct Params {
  float* out;               // PARTIALS: [splits][M][N]; PLAIN: [M][N]
  const float* bias;        // PLAIN: [N] or null
  float* residual;          // RESIDUAL: [M][N], read and written
  float* sumsq_out;         // RESIDUAL: [column blocks * splits][M]
  __nv_bfloat16* act_out;   // GATE: [M][N / 2]
  const float* x_res;       // NORM_X: residual rows [M][K]
  const float* x_sumsq;     // NORM_X: [x_parts][x_sumsq_stride]
  const float* x_weight;    // NORM_X: norm weights [K]
  int x_parts;
  int x_sumsq_stride;
  float x_eps;
  int sumsq_stride;         // RESIDUAL: row length of sumsq_out (>= M)
  int M, N, K, k_tiles, tiles_per_split, m_pad, stages;
};

__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_test_suspend(bar, parity)) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  atomicExch(&lse_gemm_error, 1);
  return false;
}

// grid: (ceil(N / BLOCK_N), 1, splits); with a cluster epilogue the `splits` blocks of a column are a cluster.
// block: 128 threads.  Dynamic shared memory: stages * (w tile [+ x tile]) [+ the block's k range of x] + barriers.
template <int BLOCK_N, bool NORM_X, int EPI>
__global__ void __launch_bounds__(128)
gemm_bf16_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                        const Params p) {
  constexpr uint32_t A_BYTES = BLOCK_N * BLOCK_K * 2;
  constexpr int ROWS_PER_WARP = BLOCK_N / 4;   // valid accumulator rows in a warp's quarter of tensor memory
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const int m_pad = p.m_pad, stages = p.stages;
  const uint32_t b_bytes = (uint32_t)m_pad * BLOCK_K * 2;
  const uint32_t stage_bytes = A_BYTES + (NORM_X ? 0u : b_bytes);
  const uint32_t x_resident = base + (uint32_t)stages * stage_bytes;                  // NORM_X: tiles_per_split x tiles
  const uint32_t bars = x_resident + (NORM_X ? (uint32_t)p.tiles_per_split * b_bytes : 0u);   // full[stages], empty[stages], accum
  const uint32_t accum_bar = bars + 16u * stages;
  unsigned char* tail = smem_raw + (accum_bar - smem_u32(smem_raw)) + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 4);
  float* inv_s = reinterpret_cast<float*>(tail + 8);                                  // NORM_X: [32] 1 / rms of each row

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BLOCK_N;
  const int split = blockIdx.z, splits = gridDim.z;
  const int tile_lo = split * p.tiles_per_split;
  const int n_tiles = max(0, min(p.k_tiles, tile_lo + p.tiles_per_split) - tile_lo);
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
  if (warp == 0) tmem_alloc(tmem_slot, tmem_cols);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t spin_limit = lse_gemm_spin_limit;
  const int withheld = lse_gemm_test_withhold ? n_tiles - 1 : -1;     // test hook: this tile never arrives

  // The weights do not depend on the kernels before this one: their first tiles are fetched at
  // once, while the kernel before may still run.  Everything that is its output (the rows of x,
  // the residual, the sums of squares) is touched after pdl_wait().
  const int early = n_tiles < stages ? n_tiles : stages;
  if (threadIdx.x == 0) {
    for (int it = 0; it < early; ++it) {
      if (it == withheld) continue;
      const uint32_t full = bars + 8u * it;
      mbar_expect_tx(full, stage_bytes);
      tma_load_2d(base + (uint32_t)it * stage_bytes, &map_w, full, (tile_lo + it) * BLOCK_K, n0);
    }
  }
  pdl_wait();
  LSE_TL_MARK(2)
  if (NORM_X) {
    // inv[m] from the producer's partial sums of squares, then this block's k range of x, tile by tile,
    // in the 128-byte-swizzled layout: row m of a tile is 128 bytes, its 16-byte chunk c lies at c ^ (m % 8).
    // All loads of a batch of chunks are issued before anything is computed (one round trip to the L2 per
    // batch, and the first batch is on its way while the sums of squares are added up).
    constexpr int BATCH = 6;
    const int chunks = n_tiles * p.M * 8;
    float4 a[BATCH][2], g[BATCH][2];
    auto locate = [&](int e, int& it, int& m, int& c, int& k) {
      it = e / (p.M * 8);
      const int rem = e % (p.M * 8);
      m = rem >> 3;
      c = rem & 7;
      k = (tile_lo + it) * BLOCK_K + c * 8;
    };
    auto load_batch = [&](int e0) {
#pragma unroll
      for (int b = 0; b < BATCH; ++b) {
        const int e = e0 + b * 128 + (int)threadIdx.x;
        int it, m, c, k;
        locate(e, it, m, c, k);
        if (e < chunks && k < p.K) {   // K is a multiple of 8: the chunk lies inside the row or beyond it
          const float* src = p.x_res + (size_t)m * p.K + k;
          a[b][0] = *reinterpret_cast<const float4*>(src);
          a[b][1] = *reinterpret_cast<const float4*>(src + 4);
          g[b][0] = *reinterpret_cast<const float4*>(p.x_weight + k);
          g[b][1] = *reinterpret_cast<const float4*>(p.x_weight + k + 4);
        } else {
          a[b][0] = a[b][1] = g[b][0] = g[b][1] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
    };
    load_batch(0);
    // inv[m]: lane l adds the parts l, l + 32, ... in order, then the lanes are added by butterfly: a fixed order
    for (int m = warp; m < p.M; m += 4) {
      float part = 0.f;
      for (int q = lane; q < p.x_parts; q += 32) part += p.x_sumsq[(size_t)q * p.x_sumsq_stride + m];
      part = warp_sum(part);
      if (lane == 0) inv_s[m] = 1.0f / sqrtf(part / (float)p.K + p.x_eps);
    }
    __syncthreads();
    for (int e0 = 0; e0 < chunks; e0 += BATCH * 128) {
      if (e0) load_batch(e0);
#pragma unroll
      for (int b = 0; b < BATCH; ++b) {
        const int e = e0 + b * 128 + (int)threadIdx.x;
        if (e >= chunks) continue;
        int it, m, c, k;
        locate(e, it, m, c, k);
        const float inv = inv_s[m];
        const __nv_bfloat162 v0 = __floats2bfloat162_rn((a[b][0].x * inv) * g[b][0].x, (a[b][0].y * inv) * g[b][0].y);
        const __nv_bfloat162 v1 = __floats2bfloat162_rn((a[b][0].z * inv) * g[b][0].z, (a[b][0].w * inv) * g[b][0].w);
        const __nv_bfloat162 v2 = __floats2bfloat162_rn((a[b][1].x * inv) * g[b][1].x, (a[b][1].y * inv) * g[b][1].y);
        const __nv_bfloat162 v3 = __floats2bfloat162_rn((a[b][1].z * inv) * g[b][1].z, (a[b][1].w * inv) * g[b][1].w);
        unsigned char* tile = base_ptr + (x_resident - base) + (size_t)it * b_bytes;
        *reinterpret_cast<uint4*>(tile + m * 128 + ((c ^ (m & 7)) << 4)) =
            make_uint4(*reinterpret_cast<const uint32_t*>(&v0), *reinterpret_cast<const uint32_t*>(&v1),
                       *reinterpret_cast<const uint32_t*>(&v2), *reinterpret_cast<const uint32_t*>(&v3));
      }
    }
    fence_async_smem();
    __syncthreads();
    LSE_TL_MARK(7)
  }

  bool issued_all = true;
  if (warp == 0) {
    if (lane == 0) {   // producer: TMA loads into the ring
      for (int it = 0; it < early && !NORM_X; ++it)
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
        if (!NORM_X) tma_load_2d(dst + A_BYTES, &map_x, full, (tile_lo + it) * BLOCK_K, 0);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {   // MMA issuer
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
        const uint32_t b_src = NORM_X ? x_resident + (uint32_t)it * b_bytes : a_src + A_BYTES;
#pragma unroll
        for (int kk = 0; kk < BLOCK_K / UMMA_K; ++kk)
          umma_bf16(tmem_base, smem_desc_k_major(a_src + kk * UMMA_K * 2), smem_desc_k_major(b_src + kk * UMMA_K * 2),
                    idesc, (it | kk) != 0 ? 1u : 0u);
        umma_commit(bars + 8u * (stages + s));   // the stage is free once these MMAs have read it
      }
      if (ok) umma_commit(accum_bar);            // the accumulator is complete
      issued_all = ok;
    }
    __syncwarp();
  }
  (void)issued_all;

  // The accumulator: warp w reads TMEM lanes 32w .. 32w+31 (rows n0 + w * ROWS_PER_WARP + lane of w), the columns
  // are the rows of x.
  const bool ready = n_tiles == 0 ? false : wait_bounded(accum_bar, 0, abort_flag, spin_limit);
  fence_after_sync();
  LSE_TL_MARK(4)
  const int n_local = warp * ROWS_PER_WARP + lane;   // row of w within the block
  const bool lane_valid = lane < ROWS_PER_WARP;

  if (EPI == PARTIALS) {
    if (ready) {
      float* dst = p.out + (size_t)split * p.M * p.N + n0 + n_local;
      for (int c0 = 0; c0 < m_pad; c0 += 8) {
        uint32_t r[8];
        tmem_ld8(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
        tmem_ld_wait();
        if (n0 + n_local < p.N && lane_valid) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (c0 + i < p.M) dst[(size_t)(c0 + i) * p.N] = __uint_as_float(r[i]);
        }
      }
    } else if (threadIdx.x == 0 && *abort_flag) {
      for (int i = 0; i < 2000; ++i) __nanosleep(100);   // let copies that may still be in flight land
    }
  } else {
    // This block's sums -> its own shared memory (the stages are free: every tile has been consumed), as
    // acc_s[m][n]; a block without tiles, or whose wait gave up, contributes zeros.
    cg::cluster_group cluster = cg::this_cluster();
    if (!ready && n_tiles > 0 && threadIdx.x == 0)
      for (int i = 0; i < 2000; ++i) __nanosleep(100);
    __syncthreads();
    float* acc_s = reinterpret_cast<float*>(base_ptr);                         // [M][BLOCK_N]
    float* sq_s = acc_s + 32 * BLOCK_N;                                       // RESIDUAL: [M][share] squares
    for (int c0 = 0; c0 < m_pad; c0 += 8) {
      uint32_t r[8];
      if (ready) {
        tmem_ld8(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) r[i] = 0u;
      }
      if (lane_valid) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (c0 + i < p.M) acc_s[(c0 + i) * BLOCK_N + n_local] = __uint_as_float(r[i]);
      }
    }
    cluster.sync();   // every block's sums are in place
    LSE_TL_MARK(5)
    const int rank = (int)cluster.block_rank();
    const float* peers[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) peers[r] = r < splits ? cluster.map_shared_rank(acc_s, r) : acc_s;
    if (EPI == GATE) {
      constexpr int HALF = BLOCK_N / 2;
      const int share = HALF / splits;            // outputs this block finishes
      const int n_out = p.N / 2;
      for (int e = threadIdx.x; e < p.M * share; e += 128) {
        const int m = e / share, o = rank * share + e % share;
        float g = 0.f, u = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r)
          if (r < splits) { g += peers[r][m * BLOCK_N + o]; u += peers[r][m * BLOCK_N + HALF + o]; }
        const int col = blockIdx.x * HALF + o;
        if (col < n_out) p.act_out[(size_t)m * n_out + col] = __float2bfloat16_rn(__fdividef(g, 1.0f + __expf(-g)) * u);
      }
    } else {
      const int share = BLOCK_N / splits;         // columns this block finishes
      for (int e = threadIdx.x; e < p.M * share; e += 128) {
        const int m = e / share, j = e % share;
        const int n = n0 + rank * share + j;
        float sum = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r)
          if (r < splits) sum += peers[r][m * BLOCK_N + rank * share + j];
        if (EPI == PLAIN) {
          if (n < p.N) p.out[(size_t)m * p.N + n] = p.bias ? sum + p.bias[n] : sum;
        } else {
          float updated = 0.f;
          if (n < p.N) {
            updated = p.residual[(size_t)m * p.N + n] + sum;
            p.residual[(size_t)m * p.N + n] = updated;
          }
          sq_s[m * share + j] = updated * updated;
        }
      }
      if (EPI == RESIDUAL) {
        __syncthreads();
        if ((int)threadIdx.x < p.M) {   // in column order: the sum does not depend on which thread squared what
          float total = 0.f;
          for (int j = 0; j < share; ++j) total += sq_s[threadIdx.x * share + j];
          p.sumsq_out[(size_t)(blockIdx.x * splits + rank) * p.sumsq_stride + threadIdx.x] = total;
        }
      }
    }
    LSE_TL_MARK(6)
    cluster.sync();   // nobody leaves while its shared memory may still be read
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
template <int BLOCK_N, bool NORM_X, int EPI>
int launch(const void* x, const void* w, Params p, int splits, int stages, cudaStream_t stream) {
  const int k_tiles = (p.K + BLOCK_K - 1) / BLOCK_K;
  if (EPI == PARTIALS) {
    splits = lse_gemm_bf16_skinny_splits(p.K, splits);
  } else {
    // the splits of a column are a cluster that shares the columns out: a power of two up to 8
    int s = 1;
    while (s * 2 <= splits && s * 2 <= 8 && s * 2 <= k_tiles) s *= 2;
    splits = s;
  }
  p.k_tiles = k_tiles;
  p.tiles_per_split = (k_tiles + splits - 1) / splits;
  const uint32_t a_bytes = (uint32_t)BLOCK_N * BLOCK_K * 2, b_bytes = (uint32_t)p.m_pad * BLOCK_K * 2;
  const uint32_t stage_bytes = a_bytes + (NORM_X ? 0u : b_bytes);
  const size_t resident = NORM_X ? (size_t)p.tiles_per_split * b_bytes : 0;
  if (stages < 2) stages = 2;
  // two blocks must fit on an SM (beside each other, or beside a block of the kernel before): at most
  // about 110 KB per block; a cluster epilogue needs room for [32][BLOCK_N] sums and as many squares
  while (stages > 2 && (size_t)stages * stage_bytes + resident + 2048 > 112 * 1024) --stages;
  if (stages > p.tiles_per_split + 1) stages = p.tiles_per_split + 1 < 2 ? 2 : p.tiles_per_split + 1;
  if (EPI != PARTIALS)
    while ((size_t)stages * stage_bytes < (size_t)2 * 32 * BLOCK_N * 4) ++stages;
  if ((size_t)stages * stage_bytes + resident + 2048 > 220 * 1024) return LSE_ERR_TOO_LARGE;
  p.stages = stages;
  const size_t smem = (size_t)stages * stage_bytes + resident + 1024 + 16 * (size_t)stages + 8 + 8 + 128 + 64;
  CUtensorMap map_w, map_x;
  if (!make_map_2d(&map_w, w, p.N, p.K, BLOCK_N)) return LSE_ERR_BAD_ARGUMENT;
  if (NORM_X) map_x = map_w;   // not used
  else if (!make_map_2d(&map_x, x, p.M, p.K, p.m_pad)) return LSE_ERR_BAD_ARGUMENT;
  static size_t configured = 0;   // largest dynamic shared memory asked for so far (per instantiation)
  if (smem > configured) {
    cudaError_t err = cudaFuncSetAttribute(gemm_bf16_skinny_kernel<BLOCK_N, NORM_X, EPI>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
    configured = smem;
  }
  dim3 grid((p.N + BLOCK_N - 1) / BLOCK_N, 1, splits);
  cudaError_t err = lse_launch_cluster(gemm_bf16_skinny_kernel<BLOCK_N, NORM_X, EPI>, grid, 128, smem, stream,
                                       EPI == PARTIALS ? 1u : (unsigned)splits, map_w, map_x, p);
  if (err != cudaSuccess) return (int)err;
  return (int)cudaGetLastError();
}

template <int BLOCK_N, bool NORM_X>
int launch_epilogue(int epilogue, const void* x, const void* w, const Params& p, int splits, int stages, cudaStream_t stream) {
  switch (epilogue) {
    case PARTIALS: return launch<BLOCK_N, NORM_X, PARTIALS>(x, w, p, splits, stages, stream);
    case PLAIN: return launch<BLOCK_N, NORM_X, PLAIN>(x, w, p, splits, stages, stream);
    case RESIDUAL: return launch<BLOCK_N, NORM_X, RESIDUAL>(x, w, p, splits, stages, stream);
    case GATE: return launch<BLOCK_N, NORM_X, GATE>(x, w, p, splits, stages, stream);
  }
  return LSE_ERR_BAD_ARGUMENT;
}
}  // namespace

// The few-rows product in all its forms.
//   x            bfloat16 [M][K], or null when the rows are made from the residual (x_res != null)
//   w            bfloat16 [N][K]
//   epilogue     0 PARTIALS: out [splits'][M][N] float32, splits' = lse_gemm_bf16_skinny_splits(K, splits)
//                1 PLAIN:    out [M][N] float32 (+ bias [N] when not null)
//                2 RESIDUAL: residual [M][N] float32 += product; sumsq_out [ceil(N / block_n) * s][sumsq_stride]
//                            where s = lse_gemm_bf16_skinny_cluster(K, splits) (partial sums of squares of the new rows)
//                3 GATE:     act_out [M][N / 2] bfloat16 = silu(gate) * up; w holds block_n / 2 gate rows, then the
//                            block_n / 2 up rows of the same outputs, and so on; N a multiple of block_n
//   x_res, x_sumsq [x_parts][x_sumsq_stride], x_weight [K], x_eps: the RMSNorm that makes x (see the top of the file)
//   block_n      rows of w per block: 128 or 64
// M <= 32 with a cluster epilogue or with x made from the residual; M <= 256 otherwise.
extern "C" int lse_gemm_bf16_skinny(const void* x, const void* w, int M, int N, int K, int splits, int stages,
                                    int block_n, int epilogue, float* out, const float* bias, float* residual,
                                    float* sumsq_out, int sumsq_stride, void* act_out, const float* x_res,
                                    const float* x_sumsq, int x_parts, int x_sumsq_stride, const float* x_weight,
                                    float x_eps, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  const int m_pad = lse_gemm_bf16_skinny_pad(M);
  const bool norm_x = x_res != nullptr;
  if (m_pad == 0 || K <= 0 || K % 8 || ((uintptr_t)w & 15)) return LSE_ERR_BAD_ARGUMENT;
  if (!norm_x && (x == nullptr || ((uintptr_t)x & 15))) return LSE_ERR_BAD_ARGUMENT;
  if (norm_x && (x_sumsq == nullptr || x_weight == nullptr || x_parts < 1 || x_sumsq_stride < M ||
                 (((uintptr_t)x_res | (uintptr_t)x_weight) & 15)))
    return LSE_ERR_BAD_ARGUMENT;
  if ((norm_x || epilogue != PARTIALS) && M > 32) return LSE_ERR_TOO_LARGE;
  if (epilogue == PARTIALS && out == nullptr) return LSE_ERR_BAD_ARGUMENT;
  if (epilogue == PLAIN && out == nullptr) return LSE_ERR_BAD_ARGUMENT;
  if (epilogue == RESIDUAL && (residual == nullptr || sumsq_out == nullptr || sumsq_stride < M)) return LSE_ERR_BAD_ARGUMENT;
  if (epilogue == GATE && (act_out == nullptr || N % block_n)) return LSE_ERR_BAD_ARGUMENT;
  Params p = {};
  p.out = out; p.bias = bias; p.residual = residual; p.sumsq_out = sumsq_out; p.act_out = (__nv_bfloat16*)act_out;
  p.x_res = x_res; p.x_sumsq = x_sumsq; p.x_weight = x_weight; p.x_parts = x_parts; p.x_sumsq_stride = x_sumsq_stride;
  p.x_eps = x_eps; p.sumsq_stride = sumsq_stride; p.M = M; p.N = N; p.K = K; p.m_pad = m_pad;
  if (block_n == 128)
    return norm_x ? launch_epilogue<128, true>(epilogue, x, w, p, splits, stages, stream)
                  : launch_epilogue<128, false>(epilogue, x, w, p, splits, stages, stream);
  if (block_n == 64)
    return norm_x ? launch_epilogue<64, true>(epilogue, x, w, p, splits, stages, stream)
                  : launch_epilogue<64, false>(epilogue, x, w, p, splits, stages, stream);
  return LSE_ERR_BAD_ARGUMENT;
}

// Blocks per column that a cluster epilogue will use for a wish of `splits`: a power of two up to 8.
extern "C" int lse_gemm_bf16_skinny_cluster(int K, int splits) {
  const int k_tiles = (K + BLOCK_K - 1) / BLOCK_K;
  int s = 1;
  while (s * 2 <= splits && s * 2 <= 8 && s * 2 <= k_tiles) s *= 2;
  return s;
}
