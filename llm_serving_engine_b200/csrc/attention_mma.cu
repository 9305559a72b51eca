// Paged attention on the tensor cores for bfloat16, head sizes 64 and 128.
//
// Two kernels share the fragment code:
//   * attn_decode_kernel: every row of the step is a single decoded token.  One
//     block = (row, kv head, split of the keys); its 4 warps walk different 16-key
//     tiles (cp.async pipeline per warp), merge in shared memory and write either
//     the result or an unnormalised partial (split-KV); the split that finishes last
//     (an arrival counter, no waiting) adds the partials up in split order.
//   * attn_prefill_kernel: portions of prompts (any mix of segment lengths).  One
//     block = (tile of consecutive rows of one request, kv head); the 64 rows of its
//     score matrix are (row, query head of the group) pairs, so the keys and values
//     of a kv head are loaded once for all its query heads; keys are walked in tiles
//     of 64 with a two-stage cp.async pipeline; causal inside the portion, all of
//     the earlier context before it.
// Scores, softmax and the output accumulation are float32 (mma.sync m16n8k16 with
// float32 accumulators; probabilities are rounded to bfloat16 for the second
// product).  Formulas as in attention_generic.cu (reference
// src/llmserve/model.py:143-176).  Cache layout: [page][kv head][offset][D].
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

LSE_TL_DEFINE(lse_timeline_attention)
LSE_CHECK_DEFINE(lse_check_attention_mma)

namespace {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  const int bytes = pred ? 16 : 0;  // 0: nothing is read, the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Transpose of an 8 x 8 matrix of 16-bit values held one 32-bit register a thread (row = lane / 4, columns 2 (lane % 4), +1).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// Byte offset of 16-byte chunk `c` of row `r` in a [rows][D] bfloat16 tile whose
// chunks are XOR-swizzled by the row, so that ldmatrix reads are conflict-free.
template <int D> __device__ __forceinline__ uint32_t tile_off(int r, int c) {
  return (uint32_t)(r * (D * 2) + ((c ^ (r & 7)) << 4));
}

constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float fast_exp2(float x) {   // 2^x, float32, 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// Copies 16 consecutive keys (rows of D bfloat16, contiguous in one cache page) of K and of V
// into two swizzled [16][D] tiles with cp.async, by NT threads (this thread is `ti`).
// Keys at or beyond `limit` (counted from the first key of the sub-tile) are zero-filled.
template <int D, int NT>
struct SubTileCopy {
  static constexpr int CH = D / 8;           // 16-byte chunks per row
  static constexpr int RPP = NT / CH;        // rows per pass
  static constexpr int PASSES = 16 / RPP;
  static_assert(NT % CH == 0 && 16 % RPP == 0, "thread count does not tile a 16-key sub-tile");
  int row0;                                  // first row this thread copies
  uint32_t lane_goff;                        // element offset of (row0, chunk) inside the 16 x D block
  uint32_t soff[PASSES];                     // byte offsets inside a swizzled tile
  __device__ __forceinline__ explicit SubTileCopy(int ti) {
    const int c = ti % CH;
    row0 = ti / CH;
    lane_goff = (uint32_t)(row0 * D + c * 8);
#pragma unroll
    for (int i = 0; i < PASSES; ++i) soff[i] = tile_off<D>(row0 + i * RPP, c);
  }
  __device__ __forceinline__ void copy(uint32_t k_dst, uint32_t v_dst, const __nv_bfloat16* k_src,
                                       const __nv_bfloat16* v_src, int limit) const {
    k_src += lane_goff;
    v_src += lane_goff;
#pragma unroll
    for (int i = 0; i < PASSES; ++i) {
      const bool valid = row0 + i * RPP < limit;
      cp_async16(k_dst + soff[i], valid ? k_src + i * RPP * D : k_src, valid);
      cp_async16(v_dst + soff[i], valid ? v_src + i * RPP * D : v_src, valid);
    }
  }
};

// ---------------------------------------------------------------------------------------------
// decode: one query row per request
// ---------------------------------------------------------------------------------------------
// Tiles of a warp in flight.  More shared memory keeps the blocks of the next kernel, which fetch their weights early,
// off the SM (measured slower at few requests); six stages for blocks that walk a whole context (64 requests, one
// split) were measured no faster either.
constexpr int DEC_STAGES = 3;
constexpr int DEC_TILE = 16;
constexpr int DEC_HEADS = 8;     // query heads of a group that a block takes: the N side of the instruction
constexpr int BT_STAGE = 1024;   // block-table entries a block keeps in shared memory

// page and offset of key j: by shift and mask when the page size is a power of two
struct PageMath {
  int size, shift;
  __device__ __forceinline__ explicit PageMath(int page_size) : size(page_size), shift(-1) {
    if ((page_size & (page_size - 1)) == 0) {
      shift = 0;
      while ((1 << shift) < page_size) ++shift;
    }
  }
  __device__ __forceinline__ int page(int j) const { return shift >= 0 ? j >> shift : j / size; }
  __device__ __forceinline__ int offset(int j) const { return shift >= 0 ? j & (size - 1) : j % size; }
};

// CLUSTER: the splits of one (row, kv head) are the blocks of a thread-block cluster and add
// themselves up through distributed shared memory; else through global partial sums and a counter.
template <int D, bool CLUSTER>
__global__ void __launch_bounds__(128)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                   const __nv_bfloat16* __restrict__ vc, __nv_bfloat16* __restrict__ out,
                   float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ arrivals,
                   const int* __restrict__ block_tables, int bt_stride,
                   const int* __restrict__ segment_of_token, const int* __restrict__ positions,
                   int n_q, int n_kv, int page_size, float scale_log2e, int num_splits, int dry_run, int num_pages,
                   int num_segments, const int* __restrict__ segment_start,
                   const int* __restrict__ segment_first_pos) {
  constexpr int CH = D / 8;                 // 16-byte chunks per row
  constexpr int TILE_BYTES = DEC_TILE * D * 2;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* q_s = smem;                                   // [16][D] bf16
  unsigned char* kv_s = smem + TILE_BYTES;                     // [warp][stage][K|V][16][D]
  __shared__ int bt_s[BT_STAGE];
  LSE_TL_BEGIN(6)
  pdl_launch_dependents();
  // The step's metadata (segments, positions, block tables) was copied to the device before the
  // step's first kernel started: it is read before waiting for the kernels that produce q, k and v.
  // blockIdx.x numbers the rows of the step, or (segment_start given: a step that also holds prompt portions) its
  // requests, of which only those that bring exactly one token are this kernel's
  const int slot = blockIdx.x;
  int t = slot;
  if (segment_start != nullptr) {
    t = segment_start[slot];
    if (segment_start[slot + 1] - t != 1) return;   // all blocks of a cluster share the request: they leave together
  }
  const int group = n_q / n_kv;
  const int gchunks = (group + DEC_HEADS - 1) / DEC_HEADS;
  const int kvh = blockIdx.y / gchunks;
  const int g0 = (blockIdx.y % gchunks) * DEC_HEADS;
  const int gcount = min(DEC_HEADS, group - g0);
  const int split = blockIdx.z;
  const int seg = LSE_CHECKED(segment_of_token[t], -1, num_segments, -1, LSE_CHECK_SEGMENT);
  if (seg < 0) return;
  const int ctx = positions[t] + 1;
  const int* bt = block_tables + (size_t)seg * bt_stride;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int first_head = kvh * group + g0;

  const int total_tiles = (ctx + DEC_TILE - 1) / DEC_TILE;
  const int per_split = (total_tiles + num_splits - 1) / num_splits;
  const int tile_lo = split * per_split;
  const int tile_hi = min(total_tiles, tile_lo + per_split);

  // this split's slice of the block table -> shared memory (one round trip instead of one per tile)
  const PageMath pm(page_size);
  const int first_page = pm.page(tile_lo * DEC_TILE);
  const int n_pages = tile_lo < tile_hi ? pm.page(min(ctx, tile_hi * DEC_TILE) - 1) - first_page + 1 : 0;
  const bool staged = n_pages <= BT_STAGE;
  if (staged)
    for (int i = tid; i < n_pages; i += 128) bt_s[i] = LSE_CHECKED(bt[first_page + i], 0, num_pages, 0, LSE_CHECK_TABLE_ENTRY);
  __syncthreads();

  unsigned char* my_s = kv_s + (size_t)warp * DEC_STAGES * 2 * TILE_BYTES;
  const uint32_t my_u32 = smem_u32(my_s);
  const bool page_tiles = (page_size % DEC_TILE) == 0 && staged;   // a 16-key tile never straddles pages
  const SubTileCopy<D, 32> copier(lane);
  auto load_tile = [&](int tile, int stage) {
    if (page_tiles) {
      const int j0 = tile * DEC_TILE;
      const int page = bt_s[pm.page(j0) - first_page];
      const size_t base = (((size_t)page * n_kv + kvh) * page_size + pm.offset(j0)) * D;
      const uint32_t k_dst = my_u32 + (uint32_t)stage * 2 * TILE_BYTES;
      copier.copy(k_dst, k_dst + TILE_BYTES, kc + base, vc + base, ctx - j0);
      return;
    }
    unsigned char* ks_ = my_s + (size_t)stage * 2 * TILE_BYTES;
    unsigned char* vs_ = ks_ + TILE_BYTES;
#pragma unroll
    for (int i = 0; i < DEC_TILE * CH / 32; ++i) {
      const int idx = i * 32 + lane;
      const int key = idx / CH, c = idx % CH;
      const int j = tile * DEC_TILE + key;
      const bool valid = j < ctx;
      size_t off = 0;
      if (valid) {
        const int logical = pm.page(j);
        const int page = staged ? bt_s[logical - first_page] : LSE_CHECKED(bt[logical], 0, num_pages, 0, LSE_CHECK_TABLE_ENTRY);
        off = (((size_t)page * n_kv + kvh) * page_size + pm.offset(j)) * D + c * 8;
      }
      cp_async16(smem_u32(ks_ + tile_off<D>(key, c)), kc + off, valid);
      cp_async16(smem_u32(vs_ + tile_off<D>(key, c)), vc + off, valid);
    }
  };

  // this warp's tiles: tile_lo + warp, + 4, ...
  const int first = tile_lo + warp;
  const int n_mine = first < tile_hi ? (tile_hi - first + 3) / 4 : 0;
  // Keys and values of earlier steps do not depend on the kernels before this one: the first tiles are
  // fetched at once, while those kernels may still run.  Only the tile that holds the row's own position
  // (its key and value were written just before this kernel) has to wait.
  // Keys that this very step writes are not fetched before the wait: the row's own position, or (a row of a prompt
  // portion: segment_first_pos given) everything from the portion's first position on.
  const int newest_tile = (segment_first_pos ? segment_first_pos[seg] : ctx - 1) / DEC_TILE;
  unsigned deferred = 0;   // stages whose tile waits
#pragma unroll
  for (int s = 0; s < DEC_STAGES; ++s) {
    if (s < n_mine) {
      if (first + 4 * s >= newest_tile) deferred |= 1u << s;
      else load_tile(first + 4 * s, s);
    }
    cp_async_commit();
  }
  // The loop over the tiles runs twice.  The first pass, before the wait for the kernels before this one,
  // works one tile through with a zero query and throws the result away: it only brings the loop's
  // instructions into the SM's instruction cache, which the other kernels of the step have emptied since
  // this one last ran (a first pass through cold code was measured at about three times a warm one).
  // `dry_run` is a kernel parameter so that the compiler keeps a single copy of the loop.
  // The keys ride the M side of the instruction (16 keys a tile), the group's heads the N side (8): S^T = K Q^T and
  // O^T = V^T P^T take half the instructions that heads on the M side (16, mostly padding) would.  A thread holds,
  // of S^T and of every 16 x 8 block of O^T, rows lane / 4 and lane / 4 + 8 and the heads 2 (lane % 4) and + 1.
  uint32_t qf[D / 16][2];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) qf[ks][0] = qf[ks][1] = 0u;
  float acc[D / 16][4];
  float m0, m1, l0, l1;    // maximum and sum of this thread's two heads (the sums over this thread's keys only)
#pragma unroll 1
  for (int pass = dry_run ? 0 : 1; pass < 2; ++pass) {
  if (pass == 1) {
    pdl_wait();
    LSE_TL_MARK(2)
    if (deferred) {   // (decoding: one warp of one split) the tiles come from the L2, and the warp waits for them here
#pragma unroll
      for (int s = 0; s < DEC_STAGES; ++s)
        if (deferred & (1u << s)) load_tile(first + 4 * s, s);
      cp_async_commit();
      cp_async_wait<0>();
    }
    // queries of the group -> shared memory (rows beyond the group are zero)
    for (int e = tid; e < 16 * CH; e += 128) {
      const int r = e / CH, c = e % CH;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < gcount) v = *reinterpret_cast<const uint4*>(q + ((size_t)t * n_q + first_head + r) * D + c * 8);
      *reinterpret_cast<uint4*>(q_s + tile_off<D>(r, c)) = v;
    }
    __syncthreads();
    {   // B operand: Q as [head][d]; one load brings the fragments of two 16-wide steps of d
#pragma unroll
      for (int ks = 0; ks < D / 16; ks += 2) {
        uint32_t r[4];
        ldmatrix_x4(r, smem_u32(q_s + tile_off<D>(lane & 7, ks * 2 + (lane >> 3))));
        qf[ks][0] = r[0]; qf[ks][1] = r[1]; qf[ks + 1][0] = r[2]; qf[ks + 1][1] = r[3];
      }
    }
    LSE_TL_MARK(4)
  }
#pragma unroll
  for (int i = 0; i < D / 16; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  m0 = m1 = -INFINITY;
  l0 = l1 = 0.f;
  const int n_run = pass == 0 ? min(n_mine, 1) : n_mine;
  for (int it = 0; it < n_run; ++it) {
    cp_async_wait<DEC_STAGES - 1>();   // all but the newest DEC_STAGES - 1 groups have landed: tile `it` is there
    __syncwarp();
    const int tile = first + 4 * it;
    const uint32_t ks_ = my_u32 + (uint32_t)(it % DEC_STAGES) * 2 * TILE_BYTES;
    const uint32_t vs_ = ks_ + TILE_BYTES;

    float s[4] = {0.f, 0.f, 0.f, 0.f}, s_odd[4] = {0.f, 0.f, 0.f, 0.f};   // even and odd steps of d add up apart: two short chains
    {
      const int mi = lane >> 3, key = (lane & 7) + (mi & 1) * 8;
#pragma unroll
      for (int ks = 0; ks < D / 16; ks += 2) {
        uint32_t a[4], b[4];
        ldmatrix_x4(a, ks_ + tile_off<D>(key, ks * 2 + (mi >> 1)));
        ldmatrix_x4(b, ks_ + tile_off<D>(key, (ks + 1) * 2 + (mi >> 1)));
        mma_bf16(s, a, qf[ks][0], qf[ks][1]);
        mma_bf16(s_odd, b, qf[ks + 1][0], qf[ks + 1][1]);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) s[e] += s_odd[e];
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int j = tile * DEC_TILE + (lane >> 2) + (e >> 1) * 8;
      s[e] = j < ctx ? s[e] * scale_log2e : -INFINITY;
    }
    // maxima of the two heads over the tile's 16 keys: this thread's two, then the lanes that hold the same heads
    float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
    }
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);   // finite: the first key of a tile lies inside the context
    const float c0 = fast_exp2(m0 - mn0), c1 = fast_exp2(m1 - mn1);
    m0 = mn0; m1 = mn1;
    const float p0 = fast_exp2(s[0] - mn0), p1 = fast_exp2(s[1] - mn1), p2 = fast_exp2(s[2] - mn0), p3 = fast_exp2(s[3] - mn1);
    l0 = l0 * c0 + (p0 + p2);
    l1 = l1 * c1 + (p1 + p3);
#pragma unroll
    for (int i = 0; i < D / 16; ++i) { acc[i][0] *= c0; acc[i][1] *= c1; acc[i][2] *= c0; acc[i][3] *= c1; }
    // P^T as the B operand: the probabilities lie as [key][head] (keys 0-7, then 8-15); transposed 8 x 8 they are
    // [head][key], a head a lane group and two neighbouring keys a register, which is what the instruction wants
    const uint32_t pb0 = movmatrix_trans(pack_bf16(p0, p1)), pb1 = movmatrix_trans(pack_bf16(p2, p3));
    {
      const int mi = lane >> 3, key = (lane & 7) + (mi >> 1) * 8;
#pragma unroll
      for (int db = 0; db < D / 16; ++db) {
        uint32_t a[4];   // V^T block [16 d][16 keys]: the tile's [key][d] pieces read transposed
        ldmatrix_x4_trans(a, vs_ + tile_off<D>(key, db * 2 + (mi & 1)));
        mma_bf16(acc[db], a, pb0, pb1);
      }
    }
    __syncwarp();
    // the stage is free: it takes the tile DEC_STAGES further on (one group per iteration, empty or not)
    if (pass == 1) {
      if (it + DEC_STAGES < n_mine) load_tile(first + 4 * (it + DEC_STAGES), it % DEC_STAGES);
      cp_async_commit();
      if (it == 0) { LSE_TL_MARK(7) }
    }
  }
  }   // pass
  cp_async_wait<0>();
  // sums of a head over the lanes that hold it
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    l0 += __shfl_xor_sync(0xffffffffu, l0, o);
    l1 += __shfl_xor_sync(0xffffffffu, l1, o);
  }
  __syncthreads();  // every warp is done with its pipeline buffers: reuse them for the merge

  float* mg_acc = reinterpret_cast<float*>(kv_s);                // [4][16][D]  (heads 0 .. 7 of the 16 are used)
  float* mg_m = mg_acc + 4 * 16 * D;                             // [4][16]
  float* mg_l = mg_m + 4 * 16;                                   // [4][16]
  {
    const int h0 = 2 * (lane & 3), h1 = h0 + 1, d0 = lane >> 2;
#pragma unroll
    for (int i = 0; i < D / 16; ++i) {
      float* a0 = mg_acc + ((size_t)warp * 16 + h0) * D + i * 16 + d0;
      float* a1 = mg_acc + ((size_t)warp * 16 + h1) * D + i * 16 + d0;
      a0[0] = acc[i][0]; a1[0] = acc[i][1]; a0[8] = acc[i][2]; a1[8] = acc[i][3];
    }
    if (lane < 4) {
      mg_m[warp * 16 + h0] = m0; mg_m[warp * 16 + h1] = m1;
      mg_l[warp * 16 + h0] = l0; mg_l[warp * 16 + h1] = l1;
    }
  }
  __syncthreads();
  // Split-KV through a cluster: block r of the cluster finishes the outputs r * push_per .. of the group's heads x D.
  __shared__ float recv_o[DEC_HEADS * 128 + 8], recv_m[8 * DEC_HEADS], recv_l[8 * DEC_HEADS];
  cg::cluster_group cluster = cg::this_cluster();
  const int push_per = (gcount * D + num_splits - 1) / num_splits;
  for (int e = tid; e < gcount * D; e += 128) {
    const int g = e / D, d = e % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, mg_m[w * 16 + g]);
    float L = 0.f, O = 0.f;
    if (M > -INFINITY) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float wgt = exp2f(mg_m[w * 16 + g] - M);
        L += mg_l[w * 16 + g] * wgt;
        O += mg_acc[((size_t)w * 16 + g) * D + d] * wgt;
      }
    }
    const int head = first_head + g;
    if (num_splits == 1) {
      out[((size_t)t * n_q + head) * D + d] = __float2bfloat16_rn(O / L);
    } else if (CLUSTER) {
      // pushed to the block of the cluster that finishes this output (its receive buffers are its own: nobody else
      // writes or reads them before the barrier); maximum and sum of a head go to every block
      const int owner = e / push_per;
      cluster.map_shared_rank(recv_o, owner)[split * push_per + e % push_per] = O;
      if (d < num_splits) {
        cluster.map_shared_rank(recv_m, d)[split * DEC_HEADS + g] = M;
        cluster.map_shared_rank(recv_l, d)[split * DEC_HEADS + g] = L;
      }
    } else {
      const size_t pidx = ((size_t)slot * n_q + head) * num_splits + split;
      part_o[pidx * D + d] = O;
      if (d == 0) { part_ml[pidx * 2] = M; part_ml[pidx * 2 + 1] = L; }
    }
  }
  LSE_TL_MARK(3)
  if (num_splits == 1) return;
  if (CLUSTER) {
    // every split has pushed its sums; after the barrier (release / acquire: the remote stores are visible) a block
    // adds up, in split order, what it received, from its own shared memory, and is free to leave
    cluster.sync();
    LSE_TL_MARK(6)
    const int rank = (int)cluster.block_rank();
    const int items = gcount * D;
    const int hi = min(items, (rank + 1) * push_per);
    for (int e = rank * push_per + tid; e < hi; e += 128) {
      const int g = e / D, d = e % D;
      float M = -INFINITY;
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < num_splits) M = fmaxf(M, recv_m[r * DEC_HEADS + g]);
      float L = 0.f, O = 0.f;
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (r < num_splits) {
          const float mr = recv_m[r * DEC_HEADS + g];
          const float w = mr == -INFINITY ? 0.f : exp2f(mr - M);
          L += recv_l[r * DEC_HEADS + g] * w;
          O += recv_o[r * push_per + (e - rank * push_per)] * w;
        }
      }
      out[((size_t)t * n_q + first_head + g) * D + d] = __float2bfloat16_rn(O / L);
    }
    LSE_TL_MARK_ANY(5, tid == 0 && blockIdx.x == 0 && blockIdx.y == 0 && rank == 0)
    return;
  }

  // The split that finishes last adds up all of them (in split order, so the sum does not depend
  // on which one that is).  `arrivals` counts finished splits per (row, block column) and is put
  // back to zero by the last one, ready for the next launch.
  __shared__ int last_flag;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int seen = atomicAdd(&arrivals[slot * gridDim.y + blockIdx.y], 1);
    last_flag = seen == num_splits - 1;
  }
  __syncthreads();
  LSE_TL_MARK_ANY(4, last_flag && tid == 0 && blockIdx.x == 0 && blockIdx.y == 0)
  if (!last_flag) return;
  __threadfence();
  // weights of the splits: w[g][sp] = 2^(m_sp - M_g) / L_g, worked out once into shared memory
  float* w_s = mg_acc;                 // [16][32]; the merge buffers are free again
  __syncthreads();
  for (int e = tid; e < gcount * 32; e += 128) {
    const int g = e >> 5, sp = e & 31;
    const size_t pbase = ((size_t)slot * n_q + first_head + g) * num_splits;
    const float m = sp < num_splits ? __ldcg(part_ml + (pbase + sp) * 2) : -INFINITY;
    const float l = sp < num_splits ? __ldcg(part_ml + (pbase + sp) * 2 + 1) : 0.f;
    // the 32 lanes of a warp hold the 32 splits of one head
    float M = m;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    const float wgt = m == -INFINITY ? 0.f : exp2f(m - M);
    float L = l * wgt;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    w_s[e] = wgt / L;
  }
  __syncthreads();
  // out[g][d] = sum_sp part_o[g][sp][d] * w[g][sp]: four d-values per thread, the loads of up to
  // eight splits issued together (splits are added in index order)
  for (int item = tid; item < gcount * (D / 4); item += 128) {
    const int g = item / (D / 4), d = (item % (D / 4)) * 4;
    const float* src = part_o + ((size_t)slot * n_q + first_head + g) * num_splits * D + d;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int sp0 = 0; sp0 < num_splits; sp0 += 8) {
      float4 v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
        v[i] = sp0 + i < num_splits ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)(sp0 + i) * D))
                                    : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float w = sp0 + i < num_splits ? w_s[g * 32 + sp0 + i] : 0.f;
        o.x += v[i].x * w; o.y += v[i].y * w; o.z += v[i].z * w; o.w += v[i].w * w;
      }
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(out + ((size_t)t * n_q + first_head + g) * D + d) = packed;
  }
  if (tid == 0) arrivals[slot * gridDim.y + blockIdx.y] = 0;
  LSE_TL_MARK_ANY(5, tid == 0 && blockIdx.x == 0 && blockIdx.y == 0)
}

// ---------------------------------------------------------------------------------------------
// prefill: tiles of consecutive rows of one request
// ---------------------------------------------------------------------------------------------
constexpr int PF_BM = 64;   // (row, head-of-group) pairs per block
constexpr int PF_BN = 64;   // keys per tile

template <int D>
__global__ void __launch_bounds__(128)
attn_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                    const __nv_bfloat16* __restrict__ vc, __nv_bfloat16* __restrict__ out,
                    const int* __restrict__ block_tables, int bt_stride,
                    const int* __restrict__ segment_start, const int* __restrict__ segment_first_pos,
                    int num_segments, int n_q, int n_kv, int page_size, float scale_log2e,
                    int rows_per_tile, int num_pages, int skip_single) {
  constexpr int CH = D / 8;
  constexpr int TILE_BYTES = PF_BN * D * 2;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* q_s = smem;                       // [64][D]
  unsigned char* kv_s = smem + PF_BM * D * 2;      // [2 stages][K|V][64][D]
  __shared__ int bt_s[BT_STAGE];
  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kvh = blockIdx.y;
  const int group = n_q / n_kv;

  // (the step's metadata is read before waiting for the kernels that produce q, k and v)
  // which tile of which request is this block's (blocks beyond the last tile leave)
  int seg, r0, cnt;
  __shared__ int tile_slot[3];
  lse_find_tile(segment_start, num_segments, rows_per_tile, skip_single, blockIdx.x, tile_slot, seg, r0, cnt);
  if (seg < 0) return;
  const int nrows = min(rows_per_tile, cnt - r0);
  const int row_base = segment_start[seg] + r0;
  const int pos0 = segment_first_pos[seg] + r0;
  const int last_pos = pos0 + nrows - 1;
  const int n_tiles = (last_pos + PF_BN) / PF_BN;
  const int* bt = block_tables + (size_t)seg * bt_stride;
  const PageMath pm(page_size);
  const int n_pages = pm.page(last_pos) + 1;
  const bool staged = n_pages <= BT_STAGE;
  if (staged)
    for (int i = tid; i < n_pages; i += 128) bt_s[i] = LSE_CHECKED(bt[i], 0, num_pages, 0, LSE_CHECK_TABLE_ENTRY);
  pdl_wait();

  for (int e = tid; e < PF_BM * CH; e += 128) {
    const int m = e / CH, c = e % CH;
    const int rl = m / group, g = m % group;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (rl < nrows) v = *reinterpret_cast<const uint4*>(q + ((size_t)(row_base + rl) * n_q + kvh * group + g) * D + c * 8);
    *reinterpret_cast<uint4*>(q_s + tile_off<D>(m, c)) = v;
  }

  const uint32_t kv_u32 = smem_u32(kv_s);
  const bool page_tiles = (page_size % 16) == 0 && staged;   // a 16-key sub-tile never straddles pages
  const SubTileCopy<D, 32> copier(lane);                      // warp w copies sub-tile w of the 64 keys
  auto load_tile = [&](int kt, int stage) {
    if (page_tiles) {
      const int j0 = kt * PF_BN + warp * 16;
      if (j0 <= last_pos) {
        const int page = bt_s[pm.page(j0)];
        const size_t base = (((size_t)page * n_kv + kvh) * page_size + pm.offset(j0)) * D;
        const uint32_t k_dst = kv_u32 + (uint32_t)stage * 2 * TILE_BYTES + (uint32_t)warp * 16 * D * 2;
        copier.copy(k_dst, k_dst + TILE_BYTES, kc + base, vc + base, last_pos + 1 - j0);
      } else {   // the whole sub-tile lies beyond the last key: zero-fill
        const uint32_t k_dst = kv_u32 + (uint32_t)stage * 2 * TILE_BYTES + (uint32_t)warp * 16 * D * 2;
        copier.copy(k_dst, k_dst + TILE_BYTES, kc, vc, 0);
      }
      return;
    }
    unsigned char* ks_ = kv_s + (size_t)stage * 2 * TILE_BYTES;
    unsigned char* vs_ = ks_ + TILE_BYTES;
#pragma unroll
    for (int i = 0; i < PF_BN * CH / 128; ++i) {
      const int idx = i * 128 + tid;
      const int key = idx / CH, c = idx % CH;
      const int j = kt * PF_BN + key;
      const bool valid = j <= last_pos;
      size_t off = 0;
      if (valid) {
        const int logical = pm.page(j);
        const int page = staged ? bt_s[logical] : LSE_CHECKED(bt[logical], 0, num_pages, 0, LSE_CHECK_TABLE_ENTRY);
        off = (((size_t)page * n_kv + kvh) * page_size + pm.offset(j)) * D + c * 8;
      }
      cp_async16(smem_u32(ks_ + tile_off<D>(key, c)), kc + off, valid);
      cp_async16(smem_u32(vs_ + tile_off<D>(key, c)), vc + off, valid);
    }
  };
  __syncthreads();   // q_s and bt_s are filled
  load_tile(0, 0);
  cp_async_commit();

  uint32_t qf[D / 16][4];
  {
    const int mi = lane >> 3, r = warp * 16 + (lane & 7) + (mi & 1) * 8;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) ldmatrix_x4(qf[ks], smem_u32(q_s + tile_off<D>(r, ks * 2 + (mi >> 1))));
  }
  // key limit of this thread's two rows
  const int ma = warp * 16 + (lane >> 2), mb = ma + 8;
  const int pos_a = pos0 + min(ma / group, nrows - 1), pos_b = pos0 + min(mb / group, nrows - 1);

  float acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  for (int kt = 0; kt < n_tiles; ++kt) {
    if (kt + 1 < n_tiles) load_tile(kt + 1, (kt + 1) & 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t ks_ = kv_u32 + (uint32_t)(kt & 1) * 2 * TILE_BYTES;
    const uint32_t vs_ = ks_ + TILE_BYTES;

    float s[PF_BN / 8][4];
#pragma unroll
    for (int i = 0; i < PF_BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    {
      const int mi = lane >> 3, key = (lane & 7) + (mi >> 1) * 8;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
        for (int nbp = 0; nbp < PF_BN / 16; ++nbp) {
          uint32_t b[4];
          ldmatrix_x4(b, ks_ + tile_off<D>(nbp * 16 + key, ks * 2 + (mi & 1)));
          mma_bf16(s[2 * nbp], qf[ks], b[0], b[1]);
          mma_bf16(s[2 * nbp + 1], qf[ks], b[2], b[3]);
        }
      }
    }
    const bool diagonal = (kt + 1) * PF_BN - 1 > pos0;   // some row of the tile ends inside these keys
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < PF_BN / 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[nb][e] * scale_log2e;
        if (diagonal) {
          const int j = kt * PF_BN + nb * 8 + (lane & 3) * 2 + (e & 1);
          if (j > ((e >> 1) ? pos_b : pos_a)) v = -INFINITY;
        }
        s[nb][e] = v;
      }
      mx0 = fmaxf(mx0, fmaxf(s[nb][0], s[nb][1]));
      mx1 = fmaxf(mx1, fmaxf(s[nb][2], s[nb][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);   // finite from the first tile on: key 0 is read by every row
    const float c0 = fast_exp2(m0 - mn0), c1 = fast_exp2(m1 - mn1);
    m0 = mn0; m1 = mn1;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int nb = 0; nb < PF_BN / 8; ++nb) {
      s[nb][0] = fast_exp2(s[nb][0] - mn0); s[nb][1] = fast_exp2(s[nb][1] - mn0);
      s[nb][2] = fast_exp2(s[nb][2] - mn1); s[nb][3] = fast_exp2(s[nb][3] - mn1);
      sum0 += s[nb][0] + s[nb][1];
      sum1 += s[nb][2] + s[nb][3];
    }
    l0 = l0 * c0 + sum0;
    l1 = l1 * c1 + sum1;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { acc[i][0] *= c0; acc[i][1] *= c0; acc[i][2] *= c1; acc[i][3] *= c1; }
    {
      const int mi = lane >> 3, key = (lane & 7) + (mi & 1) * 8;
#pragma unroll
      for (int kk = 0; kk < PF_BN / 16; ++kk) {
        uint32_t pa[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                          pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
        for (int nbp = 0; nbp < D / 16; ++nbp) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, vs_ + tile_off<D>(kk * 16 + key, nbp * 2 + (mi >> 1)));
          mma_bf16(acc[2 * nbp], pa, b[0], b[1]);
          mma_bf16(acc[2 * nbp + 1], pa, b[2], b[3]);
        }
      }
    }
    __syncthreads();   // the stage is free for the load after next
  }
  cp_async_wait<0>();
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = 1.0f / l0, inv1 = 1.0f / l1;
  const int rla = ma / group, ga = ma % group, rlb = mb / group, gb = mb % group;
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    const int d = i * 8 + (lane & 3) * 2;
    if (rla < nrows)
      *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)(row_base + rla) * n_q + kvh * group + ga) * D + d) =
          __floats2bfloat162_rn(acc[i][0] * inv0, acc[i][1] * inv0);
    if (rlb < nrows)
      *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)(row_base + rlb) * n_q + kvh * group + gb) * D + d) =
          __floats2bfloat162_rn(acc[i][2] * inv1, acc[i][3] * inv1);
  }
}

template <int D> size_t decode_smem() { return (size_t)DEC_TILE * D * 2 * (1 + 4 * DEC_STAGES * 2); }
template <int D> size_t prefill_smem() { return (size_t)PF_BM * D * 2 + (size_t)2 * 2 * PF_BN * D * 2; }

template <int D, bool CLUSTER>
int launch_decode_as(const void* q, const void* kc, const void* vc, void* out, float* part_o, float* part_ml,
                     int* arrivals, const int* block_tables, int bt_stride, const int* seg, const int* positions,
                     int tokens, int n_q, int n_kv, int page_size, float scale, int num_splits, int num_pages,
                     int num_segments, const int* segment_start, const int* segment_first_pos, cudaStream_t stream) {
  const size_t smem = decode_smem<D>();
  static bool configured = false;   // once per process: not repeated while a stream is captured
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(attn_decode_kernel<D, CLUSTER>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  const int group = n_q / n_kv;
  dim3 grid(tokens, n_kv * ((group + DEC_HEADS - 1) / DEC_HEADS), num_splits);
  cudaError_t err = lse_launch_cluster(attn_decode_kernel<D, CLUSTER>, grid, 128, smem, stream,
      CLUSTER ? (unsigned)num_splits : 1u,
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, (__nv_bfloat16*)out, part_o,
      part_ml, arrivals, block_tables, bt_stride, seg, positions, n_q, n_kv, page_size, scale * LOG2E, num_splits,
      lse_pdl_enabled ? 1 : 0, num_pages, num_segments, segment_start, segment_first_pos);
  if (err != cudaSuccess) return (int)err;
  return (int)cudaGetLastError();
}

template <int D>
int launch_decode(const void* q, const void* kc, const void* vc, void* out, float* part_o, float* part_ml,
                  int* arrivals, const int* block_tables, int bt_stride, const int* seg, const int* positions,
                  int tokens, int n_q, int n_kv, int page_size, float scale, int num_splits, int cluster,
                  int num_pages, int num_segments, const int* segment_start, const int* segment_first_pos,
                  cudaStream_t stream) {
  if (cluster && num_splits > 1 && num_splits <= 8)
    return launch_decode_as<D, true>(q, kc, vc, out, part_o, part_ml, arrivals, block_tables, bt_stride, seg, positions,
                                     tokens, n_q, n_kv, page_size, scale, num_splits, num_pages, num_segments, segment_start,
                                     segment_first_pos, stream);
  return launch_decode_as<D, false>(q, kc, vc, out, part_o, part_ml, arrivals, block_tables, bt_stride, seg, positions,
                                    tokens, n_q, n_kv, page_size, scale, num_splits, num_pages, num_segments, segment_start,
                                     segment_first_pos, stream);
}

template <int D>
int launch_prefill(const void* q, const void* kc, const void* vc, void* out, const int* block_tables,
                   int bt_stride, const int* segment_start, const int* segment_first_pos, int num_segments,
                   int tokens, int n_q, int n_kv, int page_size, float scale, int num_pages, int skip_single,
                   int max_portions, cudaStream_t stream) {
  const size_t smem = prefill_smem<D>();
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(attn_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  const int group = n_q / n_kv;
  const int rows_per_tile = PF_BM / group;
  // upper bound: every request that has tiles may end with a partial one (max_portions > 0: the caller knows that
  // at most so many requests have tiles, the others bringing single tokens that are skipped)
  const int with_tiles = (max_portions > 0 && max_portions < num_segments) ? max_portions : num_segments;
  const int tiles = (tokens + rows_per_tile - 1) / rows_per_tile + with_tiles;
  dim3 grid(tiles, n_kv);
  lse_launch(attn_prefill_kernel<D>, grid, 128, smem, stream,
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, (__nv_bfloat16*)out,
      block_tables, bt_stride, segment_start, segment_first_pos, num_segments, n_q, n_kv, page_size,
      scale * LOG2E, rows_per_tile, num_pages, skip_single);
  return (int)cudaGetLastError();
}
}  // namespace

// Whether the tensor-core kernels take this shape (else the caller uses the general kernel).
extern "C" int lse_attention_mma_supported(int head_dim, int n_q, int n_kv) {
  if (head_dim != 64 && head_dim != 128) return 0;
  if (n_kv <= 0 || n_q % n_kv) return 0;
  return (n_q / n_kv) <= PF_BM ? 1 : 0;
}

// Scratch floats that a decode launch with `num_splits` > 1 needs (outputs, then max/sum pairs).
extern "C" long long lse_attention_decode_scratch_floats(int tokens, int n_q, int head_dim, int num_splits) {
  return (long long)tokens * n_q * num_splits * (head_dim + 2);
}

// `cluster` != 0 and 2 <= num_splits <= 8: the splits form a thread-block cluster and need neither
// `scratch` nor `arrivals`.  Else `scratch` holds the partial sums and `arrivals` is tokens * n_kv *
// ceil(group / 8) ints that are zero before the first launch (the kernel leaves them zero).
// segment_first_pos != null: the rows may be rows of prompt portions (several rows of a request in one step); a row
// then fetches nothing from its request's first position of this step on before the kernels before have finished.
// segment_start != null (a step that also holds prompt portions): `tokens` counts the step's requests, block x
// of the grid is request x, and only requests that bring exactly one token are worked on (its row is
// segment_start[x]); scratch and arrivals are then sized by the number of requests.
extern "C" int lse_paged_attention_decode(const void* q, const void* k_cache, const void* v_cache, void* out,
                                          float* scratch, int* arrivals, int cluster, const int* block_tables,
                                          int bt_stride,
                                          const int* segment_of_token, const int* positions, int tokens,
                                          int n_q, int n_kv, int head_dim, int page_size, float scale,
                                          int num_splits, int num_pages, int num_segments, const int* segment_start,
                                          const int* segment_first_pos, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (!lse_attention_mma_supported(head_dim, n_q, n_kv) || page_size <= 0 || num_splits < 1 || num_splits > 32)
    return LSE_ERR_BAD_ARGUMENT;
  const bool by_cluster = cluster && num_splits > 1 && num_splits <= 8;
  if (num_splits > 1 && !by_cluster && (scratch == nullptr || arrivals == nullptr)) return LSE_ERR_BAD_ARGUMENT;
  float* part_o = scratch;
  float* part_ml = scratch ? scratch + (size_t)tokens * n_q * num_splits * head_dim : nullptr;
  if (head_dim == 128)
    return launch_decode<128>(q, k_cache, v_cache, out, part_o, part_ml, arrivals, block_tables, bt_stride,
                              segment_of_token, positions, tokens, n_q, n_kv, page_size, scale, num_splits, cluster, num_pages,
                              num_segments, segment_start, segment_first_pos, stream);
  return launch_decode<64>(q, k_cache, v_cache, out, part_o, part_ml, arrivals, block_tables, bt_stride,
                           segment_of_token, positions, tokens, n_q, n_kv, page_size, scale, num_splits, cluster, num_pages,
                           num_segments, segment_start, segment_first_pos, stream);
}

extern "C" int lse_paged_attention_prefill(const void* q, const void* k_cache, const void* v_cache, void* out,
                                           const int* block_tables, int bt_stride, const int* segment_start,
                                           const int* segment_first_pos, int num_segments, int tokens, int n_q,
                                           int n_kv, int head_dim, int page_size, float scale, int num_pages,
                                           int skip_single, int max_portions, cudaStream_t stream) {
  if (tokens <= 0 || num_segments <= 0) return 0;
  if (!lse_attention_mma_supported(head_dim, n_q, n_kv) || page_size <= 0) return LSE_ERR_BAD_ARGUMENT;
  if (head_dim == 128)
    return launch_prefill<128>(q, k_cache, v_cache, out, block_tables, bt_stride, segment_start, segment_first_pos,
                               num_segments, tokens, n_q, n_kv, page_size, scale, num_pages, skip_single, max_portions, stream);
  return launch_prefill<64>(q, k_cache, v_cache, out, block_tables, bt_stride, segment_start, segment_first_pos,
                            num_segments, tokens, n_q, n_kv, page_size, scale, num_pages, skip_single, max_portions, stream);
}
