// Paged attention for portions of prompts on the 5th-generation tensor cores
// (bfloat16, head size 64 or 128, pages of 8, 16, 32, 64 or 128 keys).
//
// One block = 128 consecutive rows of one request x one query head.  It walks the keys in
// tiles of 128 (causal: up to the position of its last row):
//
//   loader warp   TMA brings the query tile once, then the key and value tiles page by page
//                 (the block table gives the page of every 128-byte-swizzled box) into two
//                 stages each.
//   MMA warp      one thread issues  S = Q K^T  (tcgen05.mma, accumulator in tensor memory,
//                 two S buffers) and, when the probabilities of a tile are ready,  O += P V
//                 (V is the MN-major operand: its rows are keys).  S of tile j+1 is issued
//                 before P V of tile j, so the tensor cores work while the softmax runs.
//   softmax       eight warps; a thread owns half a row (64 keys) of S: tcgen05.ld, mask, row
//                 maximum (exchanged with the thread of the other half through shared memory),
//                 exp2 in float32, bfloat16 probabilities written to shared memory in the
//                 swizzled K-major layout the tensor cores read.  O stays in tensor memory and
//                 is only rescaled when a row maximum grows by more than 2^8 (the sums carry
//                 the same factor, so the quotient is exact either way); at the end
//                 O / sum is written out as bfloat16.
//
// Softmax, maxima and sums are float32.  Every wait is bounded (see tcgen05.cuh); after a
// wait that gave up the block writes nothing, frees its tensor memory and returns, and
// lse_attention_tc_status() reports it.
#include "tcgen05.cuh"

namespace {
using namespace tc;

constexpr int BM = 128;        // rows of a block
constexpr int BN = 128;        // keys per tile
constexpr int SOFTMAX_WARPS = 8;
constexpr int MMA_WARP = 8, LOADER_WARP = 9;
constexpr int THREADS = 320;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.0f;   // in powers of two
constexpr uint32_t HALF_BYTES = 128 * 128;   // a box of 128 rows x 64 bfloat16

__device__ int lse_attn_tc_error;

// Tuning builds (-DLSE_TRACE): the block of the last tile of the first request, head 0, records clock
// stamps of its first softmax thread (slots 0-5 of a tile) and of its MMA thread (slots 6, 7).
#ifdef LSE_TRACE
__device__ long long lse_attn_tc_stamps[128 * 8];
#define TC_STAMP(tile, k) if (traced && (tile) < 128) lse_attn_tc_stamps[(tile) * 8 + (k)] = clock64();
#else
#define TC_STAMP(tile, k)
#endif

enum Bar { B_Q = 0, B_KF = 1, B_KE = 3, B_VF = 5, B_VE = 7, B_SF = 9, B_SE = 11, B_PF = 13, B_OD = 14, B_COUNT = 15 };

__device__ __forceinline__ float exp2_fast(float x) {   // 2^x, 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ void pair_barrier(int quarter) {   // the two warps that share 32 rows
  asm volatile("bar.sync %0, %1;\n" ::"r"(1 + quarter), "r"(64) : "memory");
}

template <int D>
constexpr size_t attn_tc_smem() {
  return 1024 + (size_t)(D / 64) * HALF_BYTES * 5 + 2 * HALF_BYTES + 256 + 3 * 1024;
}

template <int D>
__global__ void __launch_bounds__(THREADS)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                       const int* __restrict__ block_tables, int bt_stride, const int* __restrict__ segment_start,
                       const int* __restrict__ segment_first_pos, int num_segments, int n_q, int n_kv, int page_size,
                       float scale_log2e) {
  constexpr int HALVES = D / 64;
  constexpr uint32_t Q_BYTES = HALVES * HALF_BYTES, KV_BYTES = HALVES * HALF_BYTES, P_BYTES = 2 * HALF_BYTES;
  constexpr uint32_t S_COLS = BN, O_COL = 2 * BN;
  constexpr int OD = D / 2;   // output columns of one softmax thread
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* gbase = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_s = base, k_s = q_s + Q_BYTES, v_s = k_s + 2 * KV_BYTES, p_s = v_s + 2 * KV_BYTES;
  const uint32_t bars = p_s + P_BYTES;
  unsigned char* tail = gbase + (bars - base);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + 8 * B_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 8 * B_COUNT + 4);
  float* exchange = reinterpret_cast<float*>(tail + 256);   // [2 tiles in flight][2 halves][128 rows], then sums [2][128]
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int head = blockIdx.y;
  const int kvh = head / (n_q / n_kv);
  pdl_launch_dependents();

  // which tile of which request (the step's own data: read before waiting for the kernels before);
  // blocks beyond the last tile leave.  Late tiles walk the most keys and are launched first.
  int seg = -1, r0 = 0, cnt = 0;
  {
    int before = 0;
    const int tile = gridDim.x - 1 - blockIdx.x;
    for (int s = 0; s < num_segments; ++s) {
      const int c = segment_start[s + 1] - segment_start[s];
      const int nt = (c + BM - 1) / BM;
      if (tile < before + nt) { seg = s; r0 = (tile - before) * BM; cnt = c; break; }
      before += nt;
    }
  }
  if (seg < 0) return;
  const int nrows = min(BM, cnt - r0);
  const int row_base = segment_start[seg] + r0;
  const int pos0 = segment_first_pos[seg] + r0;
  const int last_pos = pos0 + nrows - 1;
  const int n_tiles = last_pos / BN + 1;
  const int n_pages = last_pos / page_size + 1;
  const int* bt = block_tables + (size_t)seg * bt_stride;
#ifdef LSE_TRACE
  const bool traced = seg == 0 && head == 0 && r0 + BM >= cnt && (tid == 0 || tid == MMA_WARP * 32);
#endif

  if (tid == 0) {
    for (int i = 0; i < B_COUNT; ++i) mbar_init(bar(i), (i == B_SE || i == B_SE + 1 || i == B_PF) ? SOFTMAX_WARPS * 32 : 1);
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == MMA_WARP) tmem_alloc(tmem_slot, 512);   // S twice (256 columns), O (D columns)
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  int* const err = &lse_attn_tc_error;

  pdl_wait();   // queries, keys and values come from the kernel before; no bounded wait starts earlier

  if (warp == LOADER_WARP) {
    const int ppt = BN / page_size;   // pages per tile, at most 16
    if (lane == 0) {
      mbar_expect_tx(bar(B_Q), Q_BYTES);
      for (int h = 0; h < HALVES; ++h) tma_load_3d(q_s + h * HALF_BYTES, &map_q, bar(B_Q), h * 64, head, row_base);
    }
    int page_next = lane < min(ppt, n_pages) ? bt[lane] : 0;
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j & 1;
      const uint32_t parity = (uint32_t)(j >> 1) & 1u;
      const int np = min(ppt, n_pages - j * ppt);
      const int page = page_next;
      if (j + 1 < n_tiles) page_next = lane < min(ppt, n_pages - (j + 1) * ppt) ? bt[(j + 1) * ppt + lane] : 0;
      const int y = (page * n_kv + kvh) * page_size;
      const uint32_t box = (uint32_t)(lane * page_size) * 128u;
      const uint32_t bytes = (uint32_t)(np * page_size) * 128u * HALVES;
      int ok = 1;
      if (lane == 0) ok = mbar_wait(bar(B_KE + st), parity ^ 1u, abort_flag, err) ? 1 : 0;
      if (!__shfl_sync(0xffffffffu, ok, 0)) break;
      if (lane == 0) mbar_expect_tx(bar(B_KF + st), bytes);
      __syncwarp();
      if (lane < np)
        for (int h = 0; h < HALVES; ++h)
          tma_load_2d(k_s + st * KV_BYTES + h * HALF_BYTES + box, &map_k, bar(B_KF + st), h * 64, y);
      if (lane == 0) ok = mbar_wait(bar(B_VE + st), parity ^ 1u, abort_flag, err) ? 1 : 0;
      if (!__shfl_sync(0xffffffffu, ok, 0)) break;
      if (lane == 0) mbar_expect_tx(bar(B_VF + st), bytes);
      __syncwarp();
      if (lane < np)
        for (int h = 0; h < HALVES; ++h)
          tma_load_2d(v_s + st * KV_BYTES + h * HALF_BYTES + box, &map_v, bar(B_VF + st), h * 64, y);
    }
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      const uint32_t idesc_s = instr_desc_bf16(BM, BN, false, false);
      const uint32_t idesc_o = instr_desc_bf16(BM, D, false, true);
      bool ok = mbar_wait(bar(B_Q), 0, abort_flag, err);
      for (int j = 0; j <= n_tiles && ok; ++j) {
        if (j < n_tiles) {   // S_j = Q K_j^T
          const int st = j & 1;
          const uint32_t parity = (uint32_t)(j >> 1) & 1u;
          ok = mbar_wait(bar(B_KF + st), parity, abort_flag, err) && mbar_wait(bar(B_SE + st), parity ^ 1u, abort_flag, err);
          if (!ok) break;
          fence_after_sync();
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off = (uint32_t)(ks / 4) * HALF_BYTES + (uint32_t)(ks % 4) * 32u;
            umma_bf16(tmem_base + st * S_COLS, smem_desc_k_major(q_s + off),
                      smem_desc_k_major(k_s + st * KV_BYTES + off), idesc_s, ks != 0 ? 1u : 0u);
          }
          umma_commit(bar(B_KE + st));
          umma_commit(bar(B_SF + st));
          TC_STAMP(j, 6)
        }
        if (j >= 1) {        // O += P_i V_i
          const int i = j - 1, st = i & 1;
          ok = mbar_wait(bar(B_PF), (uint32_t)i & 1u, abort_flag, err) &&
               mbar_wait(bar(B_VF + st), (uint32_t)(i >> 1) & 1u, abort_flag, err);
          if (!ok) break;
          fence_after_sync();
#pragma unroll
          for (int ks = 0; ks < BN / 16; ++ks) {
            const uint32_t p_off = (uint32_t)(ks / 4) * HALF_BYTES + (uint32_t)(ks % 4) * 32u;
            umma_bf16(tmem_base + O_COL, smem_desc_k_major(p_s + p_off),
                      smem_desc_mn_major(v_s + st * KV_BYTES + (uint32_t)ks * 2048u, HALF_BYTES), idesc_o,
                      (i | ks) != 0 ? 1u : 0u);
          }
          umma_commit(bar(B_VE + st));
          umma_commit(bar(B_OD));
          TC_STAMP(i, 7)
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax
    const int quarter = warp & 3, half = warp >> 2;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int my_pos = pos0 + min(row, nrows - 1);
    float m_used = -INFINITY, l = 0.f;
    // `ok` is the same in all lanes of a warp (a vote after every wait).  A warp whose wait gave up
    // keeps meeting its partner warp at the pair barriers, which have no time limit of their own.
    bool ok = true;
    auto wait_all = [&](int which, uint32_t parity) {
      return __all_sync(0xffffffffu, mbar_wait(bar(which), parity, abort_flag, err) ? 1 : 0) != 0;
    };
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j & 1;
      uint32_t sa[32], sb[32];
      float mx = -INFINITY;
      TC_STAMP(j, 0)
      if (ok) ok = wait_all(B_SF + st, (uint32_t)(j >> 1) & 1u);
      TC_STAMP(j, 1)
      if (ok) {
        fence_after_sync();
        tmem_ld32(lane_addr + st * S_COLS + half * 64, sa);
        tmem_ld32(lane_addr + st * S_COLS + half * 64 + 32, sb);
        tmem_ld_wait();
        fence_before_sync();
        mbar_arrive(bar(B_SE + st));   // the buffer may take the tile after next
        const int kv0 = j * BN + half * 64;
        if (kv0 + 63 > my_pos) {   // the diagonal runs through these keys
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (kv0 + i > my_pos) sa[i] = 0xff800000u;
            if (kv0 + 32 + i > my_pos) sb[i] = 0xff800000u;
          }
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fmaxf(__uint_as_float(sa[i]), __uint_as_float(sb[i])));
      }
      float* slot = exchange + (j & 1) * 256;
      slot[half * 128 + row] = mx;
      pair_barrier(quarter);
      TC_STAMP(j, 2)
      if (!ok) continue;
      mx = fmaxf(mx, slot[(half ^ 1) * 128 + row]);
      const float m_new = fmaxf(m_used, mx * scale_log2e);   // finite: key 0 is visible to every row
      bool rescale = false;
      float alpha = 1.f;
      if (j == 0) {
        m_used = m_new;
      } else if (__any_sync(0xffffffffu, m_new > m_used + RESCALE_STEP)) {   // the same vote in both warps of the rows
        rescale = true;
        alpha = exp2_fast(m_used - m_new);
        m_used = m_new;
        l *= alpha;
      }
      const float neg = -m_used;
      uint32_t pk[32];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float p0 = exp2_fast(fmaf(__uint_as_float(sa[2 * i]), scale_log2e, neg));
        const float p1 = exp2_fast(fmaf(__uint_as_float(sa[2 * i + 1]), scale_log2e, neg));
        const float p2 = exp2_fast(fmaf(__uint_as_float(sb[2 * i]), scale_log2e, neg));
        const float p3 = exp2_fast(fmaf(__uint_as_float(sb[2 * i + 1]), scale_log2e, neg));
        l += (p0 + p1) + (p2 + p3);
        pk[i] = pack_bf16(p0, p1);
        pk[16 + i] = pack_bf16(p2, p3);
      }
      TC_STAMP(j, 3)
      if (j > 0) {   // P V of the tile before has read the probabilities and added to O
        ok = wait_all(B_OD, (uint32_t)(j - 1) & 1u);
        if (!ok) continue;
        fence_after_sync();
      }
      TC_STAMP(j, 4)
      if (rescale) {
#pragma unroll
        for (int c = 0; c < OD; c += 32) {
          uint32_t o[32];
          tmem_ld32(lane_addr + O_COL + half * OD + c, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(lane_addr + O_COL + half * OD + c, o);
        }
        tmem_st_wait();
      }
      // 64 probabilities = 8 chunks of 16 bytes of row `row` in the box of this half
      unsigned char* prow = gbase + (p_s - base) + half * HALF_BYTES + row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) << 4)) =
            make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      if (j == n_tiles - 1 && last_pos + 1 - j * BN < BN) {
        // rows of V beyond the last key: whatever lies there (stale keys, unwritten shared memory)
        // must not meet the zero probabilities as NaN or infinity
        ok = wait_all(B_VF + st, (uint32_t)(j >> 1) & 1u);
        if (!ok) continue;
        const int valid = last_pos + 1 - j * BN, chunks = (BN - valid) * 8;
        for (int idx = tid; idx < chunks * HALVES; idx += SOFTMAX_WARPS * 32) {
          const int h = idx / chunks, rem = idx % chunks;
          *reinterpret_cast<uint4*>(gbase + (v_s - base) + st * KV_BYTES + h * HALF_BYTES + (valid + rem / 8) * 128 + (rem % 8) * 16) =
              make_uint4(0, 0, 0, 0);
        }
      }
      fence_async_smem();
      fence_before_sync();
      mbar_arrive(bar(B_PF));
      TC_STAMP(j, 5)
    }
    if (ok) ok = wait_all(B_OD, (uint32_t)(n_tiles - 1) & 1u);
    float* sums = exchange + 512;
    sums[half * 128 + row] = l;
    pair_barrier(quarter);
    if (ok) {
      fence_after_sync();
      const float inv = 1.0f / (l + sums[(half ^ 1) * 128 + row]);
      __nv_bfloat16* dst = out + ((size_t)(row_base + row) * n_q + head) * D + half * OD;
#pragma unroll
      for (int c = 0; c < OD; c += 32) {
        uint32_t o[32];
        tmem_ld32(lane_addr + O_COL + half * OD + c, o);
        tmem_ld_wait();
        if (row < nrows) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
            w.y = pack_bf16(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
            w.z = pack_bf16(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
            w.w = pack_bf16(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c + 8 * i) = w;
          }
        }
      }
    }
  }
  if (*abort_flag && tid == 0) {
    // a wait gave up: give copies that may still be in flight time to land before the block leaves
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == MMA_WARP) tmem_dealloc(tmem_base, 512);
}

template <int D>
int launch_prefill_tc(const void* q, const void* kc, const void* vc, void* out, const int* block_tables, int bt_stride,
                      const int* segment_start, const int* segment_first_pos, int num_segments, int tokens,
                      long long num_pages, int n_q, int n_kv, int page_size, float scale, cudaStream_t stream) {
  const size_t smem = attn_tc_smem<D>();
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(attn_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  CUtensorMap map_q, map_k, map_v;
  if (!make_map_3d(&map_q, q, tokens, n_q, D, BM) ||
      !make_map_2d(&map_k, kc, num_pages * n_kv * page_size, D, page_size) ||
      !make_map_2d(&map_v, vc, num_pages * n_kv * page_size, D, page_size))
    return LSE_ERR_BAD_ARGUMENT;
  const int tiles = (tokens + BM - 1) / BM + num_segments;   // upper bound
  dim3 grid(tiles, n_q);
  cudaError_t err = lse_launch(attn_prefill_tc_kernel<D>, grid, THREADS, smem, stream, map_q, map_k, map_v,
                               (__nv_bfloat16*)out, block_tables, bt_stride, segment_start, segment_first_pos,
                               num_segments, n_q, n_kv, page_size, scale * LOG2E);
  if (err != cudaSuccess) return (int)err;
  return (int)cudaGetLastError();
}
}  // namespace

// Whether the kernel takes this shape (else the caller uses another kernel).
extern "C" int lse_attention_tc_supported(int head_dim, int n_q, int n_kv, int page_size) {
  if (head_dim != 64 && head_dim != 128) return 0;
  if (n_kv <= 0 || n_q % n_kv) return 0;
  return (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128) ? 1 : 0;
}

#ifdef LSE_TRACE
extern "C" int lse_attention_tc_stamps(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, lse_attn_tc_stamps, sizeof(long long) * 128 * 8);
}
#endif

// 0: no bounded wait has given up since the library was loaded (synchronises the device).
extern "C" int lse_attention_tc_status(void) {
  int value = 0;
  if (cudaMemcpyFromSymbol(&value, lse_attn_tc_error, sizeof(int)) != cudaSuccess) return -1;
  return value;
}

// q, out [tokens, n_q, D]; k_cache, v_cache [num_pages, n_kv, page_size, D], all bfloat16, contiguous,
// 16-byte aligned.  segment_start [S + 1]: first row of each request's portion; segment_first_pos [S]:
// the position of that row; block_tables [S, bt_stride].  Row r of a portion sees the keys 0 .. its position.
extern "C" int lse_paged_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                              const int* block_tables, int bt_stride, const int* segment_start,
                                              const int* segment_first_pos, int num_segments, int tokens,
                                              long long num_pages, int n_q, int n_kv, int head_dim, int page_size,
                                              float scale, cudaStream_t stream) {
  if (tokens <= 0 || num_segments <= 0) return 0;
  if (!lse_attention_tc_supported(head_dim, n_q, n_kv, page_size) || num_pages <= 0 || !(scale > 0.f) ||
      (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15))
    return LSE_ERR_BAD_ARGUMENT;
  if (head_dim == 128)
    return launch_prefill_tc<128>(q, k_cache, v_cache, out, block_tables, bt_stride, segment_start, segment_first_pos,
                                  num_segments, tokens, num_pages, n_q, n_kv, page_size, scale, stream);
  return launch_prefill_tc<64>(q, k_cache, v_cache, out, block_tables, bt_stride, segment_start, segment_first_pos,
                               num_segments, tokens, num_pages, n_q, n_kv, page_size, scale, stream);
}
