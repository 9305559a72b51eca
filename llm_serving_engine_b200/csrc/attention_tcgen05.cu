// Paged attention for portions of prompts on the 5th-generation tensor cores
// (bfloat16, head size 64 or 128, pages of 8, 16, 32, 64 or 128 keys).
//
// One block = 128 consecutive rows of one request x one query head.  It walks the keys in
// tiles of 128 (causal: up to the position of its last row).  The tiles go alternately to two
// groups of four softmax warps; a group has its own key and value stage, score and output
// accumulators in tensor memory, probability tile, running maxima and sums, and the two
// partial results are merged at the end.  While one group works out exponentials the other
// waits for its scores or writes probabilities, so the units of the SM overlap.
//
//   loader warp   TMA brings the query tile once, then the key and value tiles, one copy per page
//                 (the block table gives the page; a four-dimensional tensor map lays the two
//                 64-column halves of every 8 keys side by side, 128-byte swizzled), into the
//                 stage of the tile's group.
//   MMA warps     one thread issues  S = Q K^T  (tcgen05.mma, accumulator in tensor memory) for the
//                 group whose turn it is, a thread of another warp  O += P V  (V is the MN-major
//                 operand: its rows are keys), so that neither product waits behind the other's
//                 barrier.
//   softmax       a thread owns one row of its group's tiles: it reads S (tcgen05.ld), masks, finds
//                 the row maximum, takes exp2 in float32 and writes bfloat16 probabilities to shared memory in the swizzled K-major
//                 layout the tensor cores read.  After a group's first tile the probabilities
//                 are taken relative to the maximum in use, in one pass; O stays in tensor memory
//                 and is only rescaled when a row maximum has grown by more than 2^8 (the sums
//                 carry the same factor, so the quotient is exact either way).  At the end the two groups' outputs
//                 are weighted by 2^(their maximum - the common maximum), added, divided by the
//                 sum and written out as bfloat16.
//
// Softmax, maxima and sums are float32.  Every wait is bounded (see tcgen05.cuh); after a
// wait that gave up the block writes nothing, frees its tensor memory and returns, and
// lse_attention_tc_status() reports it.
#include "tcgen05.cuh"

namespace {
using namespace tc;

constexpr int BM = 128;        // rows of a block
constexpr int BN = 128;        // keys per tile
constexpr int GROUPS = 2;      // softmax groups (tiles j with j % 2 == g go to group g)
constexpr int GROUP_THREADS = 128;
constexpr int MMA_WARP = 8, LOADER_WARP = 9, PV_WARP = 10;
constexpr int THREADS = 352;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.0f;   // in powers of two
constexpr float REDO_STEP = 64.0f;
constexpr int MIN_TILES_A_PART = 4;    // a block that takes a part of a tile's keys takes at least so many key tiles
constexpr int MAX_PARTS = 8;
constexpr uint32_t HALF_BYTES = 128 * 128;   // a box of 128 rows x 64 bfloat16

__device__ int lse_attn_tc_error;
}  // namespace
LSE_CHECK_DEFINE(lse_check_attention_tc)
namespace {

// Tuning builds (-DLSE_TRACE): the block of the last tile of the first request, head 0, records clock
// stamps of the first thread of each softmax group (slots 0-5 of a tile) and of its MMA thread (6, 7).
#ifdef LSE_TRACE
__device__ long long lse_attn_tc_stamps[2 * 128 * 8];
#define TC_STAMP(tile, k) if (traced && (tile) < 128) lse_attn_tc_stamps[(tile) * 8 + (k)] = clock64();
#define TC_STAMP2(tile, k) if (traced && (tile) < 128) lse_attn_tc_stamps[1024 + (tile) * 8 + (k)] = clock64();
// start and end of every block (nanoseconds of the global timer), its SM and its number of tiles
__device__ unsigned long long lse_attn_tc_blocks[4096 * 4];
__device__ __forceinline__ unsigned long long global_ns() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ unsigned sm_id() { unsigned v; asm volatile("mov.u32 %0, %%smid;" : "=r"(v)); return v; }
#else
#define TC_STAMP(tile, k)
#define TC_STAMP2(tile, k)
#endif

// per group g: index + g
enum Bar { B_Q = 0, B_KF = 1, B_KE = 3, B_VF = 5, B_VE = 7, B_SF = 9, B_PF = 11, B_OD = 13, B_COUNT = 15 };

__device__ __forceinline__ float exp2_fast(float x) {   // 2^x, 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ void pair_barrier(int quarter) {   // the warps of the two groups that own the same 32 rows
  asm volatile("bar.sync %0, %1;\n" ::"r"(1 + quarter), "r"(64) : "memory");
}
__device__ __forceinline__ void softmax_barrier() {   // the eight softmax warps
  asm volatile("bar.sync 5, 256;\n" ::: "memory");
}
template <int D>
constexpr size_t attn_tc_smem() {
  // alignment slack, Q, a key and a value stage and a probability tile per group, barriers
  return 1024 + (size_t)(D / 64) * HALF_BYTES * (1 + 2 * GROUPS) + (size_t)GROUPS * 2 * HALF_BYTES + 256;
}

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                       const int* __restrict__ block_tables, int bt_stride, const int* __restrict__ segment_start,
                       const int* __restrict__ segment_first_pos, int num_segments, int n_q, int n_kv, int page_size,
                       float scale_log2e, int num_pages, int skip_single, int parts, float* __restrict__ scratch,
                       int* __restrict__ counters) {
  constexpr int HALVES = D / 64;
  constexpr uint32_t Q_BYTES = HALVES * HALF_BYTES, KV_BYTES = HALVES * HALF_BYTES, P_BYTES = 2 * HALF_BYTES;
  constexpr uint32_t GROUP_BYTES = HALVES * 1024;   // 8 keys (or values) in a stage: 8 rows x 128 bytes for every 64 columns
  constexpr uint32_t S_COLS = BN, O_COL = GROUPS * BN;   // tensor memory: S of group 0, S of group 1, O of group 0, O of group 1
  constexpr int OD = D / 2;   // output columns that one thread writes at the end
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* gbase = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_s = base, k_s = q_s + Q_BYTES, v_s = k_s + GROUPS * KV_BYTES, p_s = v_s + GROUPS * KV_BYTES;
  const uint32_t bars = p_s + GROUPS * P_BYTES;
  unsigned char* tail = gbase + (bars - base);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + 8 * B_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 8 * B_COUNT + 4);
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // blocks are numbered tile by tile, all heads of a tile side by side: the blocks that walk the most
  // keys (the last tiles) start first, whatever their head
  // With parts > 1 (a launch of few blocks) every tile of rows has `parts` blocks side by side, which share its keys
  // when they are many (below).
  const int head = blockIdx.x % n_q;
  const int part = (int)(blockIdx.x / n_q) % parts;
  const int rank = (int)(blockIdx.x / n_q) / parts;
  const int kvh = head / (n_q / n_kv);
  pdl_launch_dependents();

  // which tile of which request (the step's own data: read before waiting for the kernels before);
  // blocks beyond the last tile leave.  Late tiles walk the most keys and are launched first.
  int seg, r0, cnt;
  __shared__ int tile_slot[3];
  lse_find_tile(segment_start, num_segments, BM, skip_single, rank, tile_slot, seg, r0, cnt);
#ifdef LSE_TRACE
  const int block_linear = blockIdx.x;
  if (tid == 0 && block_linear < 4096) { lse_attn_tc_blocks[block_linear * 4] = global_ns(); lse_attn_tc_blocks[block_linear * 4 + 2] = sm_id(); lse_attn_tc_blocks[block_linear * 4 + 3] = 0; }
#endif
  if (seg < 0) return;
  const int nrows = min(BM, cnt - r0);
  const int row_base = segment_start[seg] + r0;
  const int pos0 = segment_first_pos[seg] + r0;
  const int last_pos = pos0 + nrows - 1;
  const int n_tiles = last_pos / BN + 1;
  const int n_pages = last_pos / page_size + 1;
  const int* bt = block_tables + (size_t)seg * bt_stride;
  // The keys of a tile of rows are shared by as many of its blocks as get MIN_TILES_A_PART key tiles each; the others
  // leave.  Every sharing block leaves its part in global memory, and the one that arrives last adds the parts up.
  const int sharing = max(1, min(parts, n_tiles / MIN_TILES_A_PART));
  if (part >= sharing) return;
  const int j_lo = (int)((long long)part * n_tiles / sharing);
  const int n_local = (int)((long long)(part + 1) * n_tiles / sharing) - j_lo;
  const int slot = rank * n_q + head;
#ifdef LSE_TRACE
  const bool traced = seg == 0 && head == 0 && r0 + BM >= cnt && (tid == 0 || tid == GROUP_THREADS || tid == MMA_WARP * 32 || tid == PV_WARP * 32);
#endif

  if (tid == 0) {
    for (int i = 0; i < B_COUNT; ++i)
      mbar_init(bar(i), (i >= B_PF && i < B_PF + 2) ? GROUP_THREADS : 1);
    *abort_flag = 0;
    *reinterpret_cast<volatile int*>(tail + 8 * B_COUNT + 12) = 1;
    mbar_init_fence();
  }
  if (warp == MMA_WARP) tmem_alloc(tmem_slot, 512);   // S and O (at most 128 columns each) of both groups
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  int* const err = &lse_attn_tc_error;

  pdl_wait();   // queries, keys and values come from the kernel before; no bounded wait starts earlier

  if (warp == LOADER_WARP) {
    // Order: K of tile j + 1 goes before V of tile j (the scores are wanted first).  A lane owns one
    // page of the tile.
    const int ppt = BN / page_size;   // pages per tile, at most 16
    if (lane == 0) {
      mbar_expect_tx(bar(B_Q), Q_BYTES);
      for (int h = 0; h < HALVES; ++h) tma_load_3d(q_s + h * HALF_BYTES, &map_q, bar(B_Q), h * 64, head, row_base);
    }
    // tiles are counted from this block's first one (jj); the keys of tile jj are those of tile j_lo + jj
    auto page_of = [&](int jj) {
      const int j = j_lo + jj;
      return (jj < n_local && lane < min(ppt, n_pages - j * ppt)) ? LSE_CHECKED(bt[j * ppt + lane], 0, num_pages, 0, LSE_CHECK_TABLE_ENTRY) : 0;
    };
    auto load = [&](int jj, int page, uint32_t dst, const CUtensorMap* map, int full, int empty) -> bool {
      const int g = jj & 1;
      const uint32_t parity = (uint32_t)(jj >> 1) & 1u;
      const int np = min(ppt, n_pages - (j_lo + jj) * ppt);
      int ok = 1;
      if (lane == 0) ok = mbar_wait(bar(empty + g), parity ^ 1u, abort_flag, err) ? 1 : 0;
      if (!__shfl_sync(0xffffffffu, ok, 0)) return false;
      if (lane == 0) mbar_expect_tx(bar(full + g), (uint32_t)(np * page_size) * 128u * HALVES);
      __syncwarp();
      if (lane < np)   // one copy per page: its groups of 8 keys, the two halves of the head size side by side
        tma_load_4d(dst + g * KV_BYTES + (uint32_t)(lane * page_size) * 128u * HALVES, map, bar(full + g), 0, 0, 0,
                    (page * n_kv + kvh) * (page_size / 8));
      return true;
    };
    int page_k = page_of(0), page_v = page_k;
    bool ok = load(0, page_k, k_s, &map_k, B_KF, B_KE);
    for (int jj = 0; jj < n_local && ok; ++jj) {
      page_k = page_of(jj + 1);
      if (jj + 1 < n_local) ok = load(jj + 1, page_k, k_s, &map_k, B_KF, B_KE);
      if (ok) ok = load(jj, page_v, v_s, &map_v, B_VF, B_VE);
      page_v = page_k;
    }
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      // S_j = Q K_j^T as soon as the group of tile j has read the scores of its tile before (it has, when
      // its probabilities are written).  The keys are waited for first: they have long arrived, and the
      // wait that matters then comes last.
      const uint32_t idesc_s = instr_desc_bf16(BM, BN, false, false);
      bool ok = mbar_poll(bar(B_Q), 0, abort_flag, err);
      for (int j = 0; j < n_local && ok; ++j) {
        const int g = j & 1;
        const uint32_t parity = (uint32_t)(j >> 1) & 1u;
        TC_STAMP2(j, 1)
        ok = mbar_poll(bar(B_KF + g), parity, abort_flag, err);
        TC_STAMP2(j, 2)
        if (ok && j >= GROUPS) ok = mbar_poll(bar(B_PF + g), parity ^ 1u, abort_flag, err);
        if (!ok) break;
        fence_after_sync();
        TC_STAMP2(j, 6)
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (uint32_t)(ks / 4) * HALF_BYTES + (uint32_t)(ks % 4) * 32u;
          const uint32_t k_off = (uint32_t)(ks / 4) * 1024u + (uint32_t)(ks % 4) * 32u;
          umma_bf16(tmem_base + g * S_COLS, smem_desc_k_major(q_s + off),
                    smem_desc_k_major(k_s + g * KV_BYTES + k_off, GROUP_BYTES), idesc_s, ks != 0 ? 1u : 0u);
        }
        TC_STAMP2(j, 7)
        umma_commit(bar(B_KE + g));
        umma_commit(bar(B_SF + g));
        TC_STAMP(j, 6)
      }
    }
    __syncwarp();
  } else if (warp == PV_WARP) {
    if (lane == 0) {
      // O_g += P_i V_i as soon as the probabilities of tile i are written
      const uint32_t idesc_o = instr_desc_bf16(BM, D, false, true);
      bool ok = true;
      for (int i = 0; i < n_local && ok; ++i) {
        const int g = i & 1;
        const uint32_t parity = (uint32_t)(i >> 1) & 1u;
        TC_STAMP2(i, 0)
        // (Letting the scores of the group's next tile go first, which the group waits for sooner than for this
        // product, was slower on long prompts: 214 against 208 ms for 30,720 tokens.)
        ok = mbar_poll(bar(B_VF + g), parity, abort_flag, err) && mbar_poll(bar(B_PF + g), parity, abort_flag, err);
        if (!ok) break;
        fence_after_sync();
        TC_STAMP2(i, 3)
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
          const uint32_t p_off = (uint32_t)(ks / 4) * HALF_BYTES + (uint32_t)(ks % 4) * 32u;
          umma_bf16(tmem_base + O_COL + g * D, smem_desc_k_major(p_s + g * P_BYTES + p_off),
                    smem_desc_mn_major(v_s + g * KV_BYTES + (uint32_t)ks * 2u * GROUP_BYTES, 1024u, GROUP_BYTES), idesc_o,
                    (i >= GROUPS || ks != 0) ? 1u : 0u);
        }
        TC_STAMP2(i, 4)
        umma_commit(bar(B_VE + g));
        umma_commit(bar(B_OD + g));
        TC_STAMP2(i, 5)
        TC_STAMP(i, 7)
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax
    const int g = warp >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t s_addr = lane_addr + g * S_COLS, o_addr = lane_addr + O_COL + g * D;
    const int my_pos = pos0 + min(row, nrows - 1);
    unsigned char* prow = gbase + (p_s - base) + g * P_BYTES + row * 128;
    float m_used = -INFINITY, m_seen = -INFINITY, l = 0.f;   // the maximum that O and l are relative to; the largest score seen
    bool pending = false;                                    // m_seen has outgrown m_used: O and l are to be rescaled
    // `ok` is the same in all lanes of a warp (a vote after every wait).  A warp whose wait gave up
    // still meets the warp of the other group at the pair barrier, which has no time limit of its own.
    bool ok = true;
    auto wait_all = [&](int which, uint32_t parity) {
      const bool done = mbar_test(bar(which), parity) || mbar_wait(bar(which), parity, abort_flag, err);
      return __all_sync(0xffffffffu, done ? 1 : 0) != 0;
    };
    for (int j = g; j < n_local && ok; j += GROUPS) {   // j counts this block's tiles
      const uint32_t parity = (uint32_t)(j >> 1) & 1u;
      TC_STAMP(j, 0)
      ok = wait_all(B_SF + g, parity);
      if (!ok) break;
      TC_STAMP(j, 1)
      fence_after_sync();
      const int kv0 = (j_lo + j) * BN;
      const bool diagonal = kv0 + BN - 1 > my_pos;   // some keys of this tile lie beyond this row's position
      const bool first = j < GROUPS;                 // this group's first tile
      bool rescale = false;
      float alpha = 1.f;
      if (first) {
        // the row maximum of the first tile is found before anything is exponentiated
        float mx = -INFINITY;
#pragma unroll
        for (int c = 0; c < BN; c += 32) {
          uint32_t s[32];
          tmem_ld32(s_addr + c, s);
          tmem_ld_wait();
          if (diagonal) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (kv0 + c + i > my_pos) s[i] = 0xff800000u;
          }
#pragma unroll
          for (int i = 0; i < 32; i += 2) mx = fmaxf(mx, fmaxf(__uint_as_float(s[i]), __uint_as_float(s[i + 1])));
        }
        // a row of tile 0 always sees key 0; a row's last tile may be hidden entirely (-inf: nothing is added then)
        m_used = m_seen = mx * scale_log2e;
      } else if (pending) {   // the tile before raised the maximum by more than the step: O and the sum follow now
        rescale = true;
        alpha = m_used == -INFINITY ? 0.f : exp2_fast(m_used - m_seen);
        m_used = m_seen;
        l *= alpha;
        pending = false;
      }
      TC_STAMP(j, 2)
      if (j >= GROUPS) {   // P V of this group's tile before has read the probabilities and added to O
        ok = wait_all(B_OD + g, parity ^ 1u);
        if (!ok) break;
        fence_after_sync();
      }
      TC_STAMP(j, 3)
      // Later tiles take their probabilities relative to the maximum in use, in one pass, and find their
      // own maximum on the way.  A maximum that grew by more than 2^8 is taken over before the next
      // tile; one that grew by more than 2^64 (bfloat16 and float32 would run out of range a little
      // further on) is taken over at once and the tile is done again.
#pragma unroll 1
      for (int attempt = 0; attempt < 2; ++attempt) {
        if (rescale) {
#pragma unroll
          for (int c = 0; c < D; c += 32) {
            uint32_t o[32];
            tmem_ld32(o_addr + c, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(o_addr + c, o);
          }
          tmem_st_wait();
          rescale = false;
        }
        const float neg = m_used == -INFINITY ? 0.f : -m_used;   // every score is -inf then as well: p = 0
        float mx = -INFINITY, sum = 0.f;
        // 32 keys = 4 chunks of 16 bytes at a time; the next 32 scores are on their way from tensor memory
        // while these are worked on
        auto take = [&](uint32_t (&s)[32], int c) {
          if (diagonal) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (kv0 + c + i > my_pos) s[i] = 0xff800000u;
          }
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            const float s0 = __uint_as_float(s[2 * i]), s1 = __uint_as_float(s[2 * i + 1]);
            const float s2 = __uint_as_float(s[2 * i + 2]), s3 = __uint_as_float(s[2 * i + 3]);
            mx = fmaxf(mx, fmaxf(fmaxf(s0, s1), fmaxf(s2, s3)));
            float p0 = fmaf(s0, scale_log2e, neg), p1 = fmaf(s1, scale_log2e, neg);
            float p2 = fmaf(s2, scale_log2e, neg), p3 = fmaf(s3, scale_log2e, neg);
            p0 = exp2_fast(p0); p1 = exp2_fast(p1); p2 = exp2_fast(p2); p3 = exp2_fast(p3);
            sum += (p0 + p1) + (p2 + p3);
            pk[i] = pack_bf16(p0, p1);
            pk[i + 1] = pack_bf16(p2, p3);
          }
          unsigned char* box = prow + (c / 64) * HALF_BYTES;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int chunk = (c % 64) / 8 + k;
            *reinterpret_cast<uint4*>(box + ((chunk ^ (row & 7)) << 4)) = make_uint4(pk[4 * k], pk[4 * k + 1], pk[4 * k + 2], pk[4 * k + 3]);
          }
        };
        uint32_t sa[32], sb[32];
        tmem_ld32(s_addr, sa);
#pragma unroll
        for (int c = 0; c < BN; c += 64) {
          tmem_ld_wait();
          tmem_ld32(s_addr + c + 32, sb);
          take(sa, c);
          tmem_ld_wait();
          if (c + 64 < BN) tmem_ld32(s_addr + c + 64, sa);
          take(sb, c + 32);
        }
        const float m_tile = mx * scale_log2e;
        if (first || !__any_sync(0xffffffffu, m_tile > m_used + REDO_STEP)) {
          l += sum;
          m_seen = fmaxf(m_seen, m_tile);
          pending = __any_sync(0xffffffffu, m_seen > m_used + RESCALE_STEP) != 0;
          break;
        }
        rescale = true;
        alpha = m_used == -INFINITY ? 0.f : exp2_fast(m_used - fmaxf(m_used, m_tile));
        m_used = fmaxf(m_used, m_tile);
        m_seen = fmaxf(m_seen, m_used);
        l *= alpha;
      }
      TC_STAMP(j, 4)
      if (j_lo + j == n_tiles - 1 && last_pos + 1 - kv0 < BN) {
        // rows of V beyond the last key: whatever lies there (stale keys, unwritten shared memory)
        // must not meet the zero probabilities as NaN or infinity
        ok = wait_all(B_VF + g, parity);
        if (!ok) break;
        const int valid = last_pos + 1 - kv0, chunks = (BN - valid) * 8;
        for (int idx = tid - g * GROUP_THREADS; idx < chunks * HALVES; idx += GROUP_THREADS) {
          const int h = idx / chunks, rem = idx % chunks;
          const int r = valid + rem / 8;
          *reinterpret_cast<uint4*>(gbase + (v_s - base) + g * KV_BYTES + (r / 8) * GROUP_BYTES + h * 1024 + (r % 8) * 128 + (rem % 8) * 16) =
              make_uint4(0, 0, 0, 0);
        }
      }
      fence_async_smem();
      fence_before_sync();
      mbar_arrive(bar(B_PF + g));
      TC_STAMP(j, 5)
    }
    // ---------------------------------------------------------------- merge of the two groups
    // A group hands its maxima and sums over in its own key stage: the group has seen the scores of
    // its last tile, so nothing reads or writes that stage any more.
    float* mine = reinterpret_cast<float*>(gbase + (k_s - base) + g * KV_BYTES);
    const float* other = reinterpret_cast<const float*>(gbase + (k_s - base) + (g ^ 1) * KV_BYTES);
    mine[row] = m_used;
    mine[128 + row] = l;
    pair_barrier(quarter);
    const float m_other = other[row], l_other = other[128 + row];
    const float m_all = fmaxf(m_used, m_other);                      // finite when the block holds key 0
    const float w_mine = m_used == -INFINITY ? 0.f : exp2_fast(m_used - m_all);
    const float w_other = m_other == -INFINITY ? 0.f : exp2_fast(m_other - m_all);
    // group 0's term first in both groups' threads: the two threads of a row hold the same bits
    const float l_all = g == 0 ? fmaf(l_other, w_other, l * w_mine) : fmaf(l, w_mine, l_other * w_other);
    // a block that holds all keys of its rows divides by the sum here; one that holds a part of them leaves its
    // output relative to its own maximum, undivided
    const bool shared = sharing > 1;
    const float inv = shared ? 1.0f : 1.0f / l_all;
    const float w0 = (g == 0 ? w_mine : w_other) * inv, w1 = (g == 0 ? w_other : w_mine) * inv;
    // both groups' last products must have landed (group 1 has none when there is a single tile)
    const int n0 = (n_local + 1) / 2, n1 = n_local / 2;
    if (ok) ok = wait_all(B_OD + 0, (uint32_t)(n0 - 1) & 1u);
    if (ok && n1 > 0) ok = wait_all(B_OD + 1, (uint32_t)(n1 - 1) & 1u);
    // this thread owns columns g * D/2 .. of its row: the same columns of both groups' outputs
    __nv_bfloat16* dst = out + ((size_t)(row_base + row) * n_q + head) * D + g * OD;
    if (!shared) {
      if (ok) {
        fence_after_sync();
#pragma unroll
        for (int c = 0; c < OD; c += 32) {
          uint32_t a[32], b[32];
          tmem_ld32(lane_addr + O_COL + g * OD + c, a);
          if (n1 > 0) tmem_ld32(lane_addr + O_COL + D + g * OD + c, b);
          tmem_ld_wait();
          if (row < nrows) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float v[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                v[e] = __uint_as_float(a[8 * i + e]) * w0;
                if (n1 > 0) v[e] = fmaf(__uint_as_float(b[8 * i + e]), w1, v[e]);
              }
              *reinterpret_cast<uint4*>(dst + c + 8 * i) =
                  make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
            }
          }
        }
      }
    } else {
      // ------------------------------------------------------------ several blocks, one tile of rows
      // Each block leaves its part in global memory: output as [D / 4][BM] groups of four columns (a warp's rows side
      // by side), maxima [BM], sums [BM], float32.  The block that finds all other parts there adds them up, the
      // parts in their order whoever adds, and writes the rows.  No block waits for another.  A block whose wait
      // gave up leaves nothing and does not count itself: the rows are then never written, and the status word says so.
      constexpr int PART_FLOATS = BM * D + 2 * BM;
      float* const parts_base = scratch + (size_t)slot * MAX_PARTS * PART_FLOATS;
      float* const my_part = parts_base + (size_t)part * PART_FLOATS;
      volatile int* const arrived = reinterpret_cast<volatile int*>(tail + 8 * B_COUNT + 8);
      volatile int* const whole = reinterpret_cast<volatile int*>(tail + 8 * B_COUNT + 12);   // 1 until a warp's wait gave up
      if (ok) {
        fence_after_sync();
#pragma unroll
        for (int c = 0; c < OD; c += 32) {
          uint32_t a[32], b[32];
          tmem_ld32(lane_addr + O_COL + g * OD + c, a);
          if (n1 > 0) tmem_ld32(lane_addr + O_COL + D + g * OD + c, b);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float v[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              v[e] = __uint_as_float(a[4 * i + e]) * w0;
              if (n1 > 0) v[e] = fmaf(__uint_as_float(b[4 * i + e]), w1, v[e]);
            }
            reinterpret_cast<float4*>(my_part)[((g * OD + c) / 4 + i) * BM + row] = make_float4(v[0], v[1], v[2], v[3]);
          }
        }
        if (g == 0) { my_part[BM * D + row] = m_all; my_part[BM * D + BM + row] = l_all; }
        __threadfence();
      }
      if (!ok) *whole = 0;
      softmax_barrier();
      if (tid == 0) *arrived = *whole ? atomicAdd(counters + slot, 1) : -1;
      softmax_barrier();
      if (*arrived == sharing - 1) {   // all other parts are there
        __threadfence();
        float m_parts[MAX_PARTS], m_tile = -INFINITY;
#pragma unroll
        for (int p = 0; p < MAX_PARTS; ++p) {
          m_parts[p] = p < sharing ? __ldcg(parts_base + (size_t)p * PART_FLOATS + BM * D + row) : -INFINITY;
          m_tile = fmaxf(m_tile, m_parts[p]);
        }
        float sum = 0.f, weight[MAX_PARTS];
#pragma unroll
        for (int p = 0; p < MAX_PARTS; ++p) {
          weight[p] = (p < sharing && m_parts[p] != -INFINITY) ? exp2_fast(m_parts[p] - m_tile) : 0.f;
          if (p < sharing) sum = fmaf(__ldcg(parts_base + (size_t)p * PART_FLOATS + BM * D + BM + row), weight[p], sum);
        }
        const float inv_sum = 1.0f / sum;
        if (row < nrows) {
#pragma unroll 2
          for (int c = 0; c < OD; c += 8) {
            float4 x0 = make_float4(0.f, 0.f, 0.f, 0.f), x1 = x0;
#pragma unroll
            for (int p = 0; p < MAX_PARTS; ++p) {
              if (p < sharing) {
                const float4* src = reinterpret_cast<const float4*>(parts_base + (size_t)p * PART_FLOATS) + ((g * OD + c) / 4) * BM + row;
                const float4 y0 = __ldcg(src), y1 = __ldcg(src + BM);
                const float w = weight[p];
                x0.x = fmaf(y0.x, w, x0.x); x0.y = fmaf(y0.y, w, x0.y); x0.z = fmaf(y0.z, w, x0.z); x0.w = fmaf(y0.w, w, x0.w);
                x1.x = fmaf(y1.x, w, x1.x); x1.y = fmaf(y1.y, w, x1.y); x1.z = fmaf(y1.z, w, x1.z); x1.w = fmaf(y1.w, w, x1.w);
              }
            }
            *reinterpret_cast<uint4*>(dst + c) = make_uint4(
                pack_bf16(x0.x * inv_sum, x0.y * inv_sum), pack_bf16(x0.z * inv_sum, x0.w * inv_sum),
                pack_bf16(x1.x * inv_sum, x1.y * inv_sum), pack_bf16(x1.z * inv_sum, x1.w * inv_sum));
          }
        }
        if (tid == 0) counters[slot] = 0;   // as the next launch expects it
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
#ifdef LSE_TRACE
  if (tid == 0 && block_linear < 4096) { lse_attn_tc_blocks[block_linear * 4 + 1] = global_ns(); lse_attn_tc_blocks[block_linear * 4 + 3] = n_local; }
#endif
}

template <int D>
int launch_prefill_tc(const void* q, const void* kc, const void* vc, void* out, const int* block_tables, int bt_stride,
                      const int* segment_start, const int* segment_first_pos, int num_segments, int tokens,
                      long long num_pages, int n_q, int n_kv, int page_size, float scale, int skip_single,
                      int max_portions, float* scratch, int* counters, long long scratch_slots, cudaStream_t stream) {
  const size_t smem = attn_tc_smem<D>();
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(attn_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  CUtensorMap map_q, map_k, map_v;
  if (!make_map_3d(&map_q, q, tokens, n_q, D, BM) ||
      !make_map_row_groups(&map_k, kc, num_pages * n_kv * page_size, D, page_size) ||
      !make_map_row_groups(&map_v, vc, num_pages * n_kv * page_size, D, page_size))
    return LSE_ERR_BAD_ARGUMENT;
  // upper bound: every request that has tiles may end with a partial one (max_portions > 0: the caller knows that
  // at most so many requests have tiles, the others bringing single tokens that are skipped)
  const int with_tiles = (max_portions > 0 && max_portions < num_segments) ? max_portions : num_segments;
  const int tiles = (tokens + BM - 1) / BM + with_tiles;
  // With fewer blocks than SMs, several blocks share the keys of a tile of rows (the kernel decides tile by tile how
  // many: a part is at least MIN_TILES_A_PART key tiles).  The parts meet in `scratch`.
  static int sm_count = 0;
  if (sm_count == 0) {
    int device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
  }
  const long long blocks = (long long)tiles * n_q;
  int parts = 1;
  if (scratch != nullptr && counters != nullptr && blocks <= scratch_slots) {
    parts = (int)((5LL * sm_count) / (4 * blocks));
    parts = parts < 1 ? 1 : (parts > MAX_PARTS ? MAX_PARTS : parts);
  }
  dim3 grid((unsigned)(blocks * parts));
  cudaError_t err = lse_launch(attn_prefill_tc_kernel<D>, grid, THREADS, smem, stream, map_q, map_k, map_v,
                               (__nv_bfloat16*)out, block_tables, bt_stride, segment_start, segment_first_pos,
                               num_segments, n_q, n_kv, page_size, scale * LOG2E, (int)num_pages, skip_single, parts,
                               scratch, counters);
  if (err != cudaSuccess) return (int)err;
  return (int)cudaGetLastError();
}
}  // namespace

// Values of float32 scratch per slot (a tile of rows of one head: up to MAX_PARTS parts).  scratch (scratch_slots
// times that) and counters (int32, scratch_slots, zero; the kernel leaves them zero) may be null: they let several
// blocks share the keys of a tile of rows when a launch has fewer blocks than the GPU has SMs.
extern "C" int lse_attention_tc_scratch_floats(void) { return MAX_PARTS * (BM * 128 + 2 * BM); }

// Whether the kernel takes this shape (else the caller uses another kernel).
extern "C" int lse_attention_tc_supported(int head_dim, int n_q, int n_kv, int page_size) {
  if (head_dim != 64 && head_dim != 128) return 0;
  if (n_kv <= 0 || n_q % n_kv) return 0;
  return (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128) ? 1 : 0;
}

#ifdef LSE_TRACE
extern "C" int lse_attention_tc_blocks(unsigned long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, lse_attn_tc_blocks, sizeof(unsigned long long) * 4096 * 4);
}
extern "C" int lse_attention_tc_stamps(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, lse_attn_tc_stamps, sizeof(long long) * 2 * 128 * 8);
}
#endif

// 0: no bounded wait has given up since the library was loaded (synchronises the device).
extern "C" int lse_attention_tc_status(void) {
  int value = 0;
  if (cudaMemcpyFromSymbol(&value, lse_attn_tc_error, sizeof(int)) != cudaSuccess) return -1;
  return value;
}

// Queue a copy of the word to `host_dst` (pinned) on `stream`: the host reads it with the step's tokens,
// without a synchronisation of its own.
extern "C" int lse_attention_tc_status_async(int* host_dst, cudaStream_t stream) {
  return (int)cudaMemcpyFromSymbolAsync(host_dst, lse_attn_tc_error, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
}
extern "C" int lse_attention_tc_status_reset(void) {
  const int zero = 0;
  return (int)cudaMemcpyToSymbol(lse_attn_tc_error, &zero, sizeof(int));
}

// q, out [tokens, n_q, D]; k_cache, v_cache [num_pages, n_kv, page_size, D], all bfloat16, contiguous,
// 16-byte aligned.  segment_start [S + 1]: first row of each request's portion; segment_first_pos [S]:
// the position of that row; block_tables [S, bt_stride].  Row r of a portion sees the keys 0 .. its position.
extern "C" int lse_paged_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                              const int* block_tables, int bt_stride, const int* segment_start,
                                              const int* segment_first_pos, int num_segments, int tokens,
                                              long long num_pages, int n_q, int n_kv, int head_dim, int page_size,
                                              float scale, int skip_single, int max_portions, float* scratch,
                                              int* counters, long long scratch_slots, cudaStream_t stream) {
  if (tokens <= 0 || num_segments <= 0) return 0;
  if (!lse_attention_tc_supported(head_dim, n_q, n_kv, page_size) || num_pages <= 0 || !(scale > 0.f) ||
      (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15))
    return LSE_ERR_BAD_ARGUMENT;
  if (head_dim == 128)
    return launch_prefill_tc<128>(q, k_cache, v_cache, out, block_tables, bt_stride, segment_start, segment_first_pos,
                                  num_segments, tokens, num_pages, n_q, n_kv, page_size, scale, skip_single, max_portions, scratch,
                                  counters, scratch_slots, stream);
  return launch_prefill_tc<64>(q, k_cache, v_cache, out, block_tables, bt_stride, segment_start, segment_first_pos,
                               num_segments, tokens, num_pages, n_q, n_kv, page_size, scale, skip_single, max_portions, scratch,
                                  counters, scratch_slots, stream);
}
