// Row-wise kernels of the decoder: embedding gather, RMSNorm fused with the
// residual sum, rotary position encoding fused with the bias and the write into
// the paged cache, and the SiLU gate.  Formulas follow the reference project's
// src/llmserve/model.py (RMSNorm :20-23, rotary :29-43, MLP :188).
//
// An input that comes from a matrix product may be given as a stack of
// `n_partials` float32 partial sums (split-K), `partial_stride` elements apart;
// the kernels add them in index order before anything else, so the sum is the
// same whatever else runs.
#include "common.cuh"

LSE_TL_DEFINE(lse_timeline_elementwise)
LSE_CHECK_DEFINE(lse_check_elementwise)

// ------------------------------------------------------------------ embedding
// residual[t, :] = float(table[ids[t], :])
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ out, int hidden, int vocab) {
  LSE_TL_BEGIN(1)
  pdl_launch_dependents();
  pdl_wait();
  LSE_TL_MARK(2)
  const int t = blockIdx.x;
  const int id = LSE_CHECKED(ids[t], 0, vocab, -1, LSE_CHECK_TOKEN_ID);
  float* dst = out + (size_t)t * hidden;
  if (id < 0 || id >= vocab) {  // padding row of a fixed-shape batch
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.f;
    return;
  }
  const T* src = table + (size_t)id * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32<T>(src[i]);
  LSE_TL_MARK(3)
}

extern "C" int lse_embedding(const void* table, int table_dtype, const int* ids, float* out,
                             int tokens, int hidden, int vocab, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (table_dtype == LSE_DTYPE_F32)
    lse_launch(embedding_kernel<float>, tokens, threads, 0, stream, (const float*)table, ids, out, hidden, vocab);
  else if (table_dtype == LSE_DTYPE_BF16)
    lse_launch(embedding_kernel<__nv_bfloat16>, tokens, threads, 0, stream, (const __nv_bfloat16*)table, ids, out, hidden, vocab);
  else
    return LSE_ERR_BAD_ARGUMENT;
  LSE_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ add + RMSNorm
// For output row r (source row s = rows ? rows[r] : r):
//   x = residual[s] + sum_p float(delta[p][s])   (delta may be null)
//   if write_residual: residual[s] = x           (float32 residual stream)
//   out[r] = (x * rsqrt(mean(x^2) + eps)) * weight
template <typename TD> __device__ __forceinline__ void load4(const TD* p, float (&v)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
  v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
template <typename TO> __device__ __forceinline__ void store4(TO* p, const float (&v)[4]);
template <> __device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<uint32_t*>(&a);
  t.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = t;
}

constexpr int NORM_THREADS = 512;
constexpr int NORM_CHUNKS = 4;   // float4 chunks a thread keeps: hidden <= 512 * 4 * 4 = 8192

// One pass: the row stays in registers between the sum of squares and the scaling.
// hidden % 4 == 0 and hidden <= NORM_THREADS * NORM_CHUNKS * 4.
template <typename TD, typename TO>
__global__ void __launch_bounds__(NORM_THREADS)
add_rmsnorm_vec_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int n_partials,
                       long long partial_stride, const float* __restrict__ weight, TO* __restrict__ out,
                       const int* __restrict__ rows, int hidden, float eps, int write_residual, int source_rows) {
  LSE_TL_BEGIN(2)
  pdl_launch_dependents();
  __shared__ float scratch[32];
  const int chunks = hidden >> 2;
  // the norm weights do not depend on earlier kernels: fetch them before waiting for those
  float w[NORM_CHUNKS][4];
#pragma unroll
  for (int c = 0; c < NORM_CHUNKS; ++c) {
    const int i = (c * (int)blockDim.x + threadIdx.x);
    if (i < chunks) load4<float>(weight + 4 * i, w[c]);
  }
  pdl_wait();
  LSE_TL_MARK(2)
  const int r = blockIdx.x;
  const int s = rows ? LSE_CHECKED(rows[r], -1, source_rows, -1, LSE_CHECK_ROW) : r;
  if (s < 0) return;
  float* res = residual + (size_t)s * hidden;
  const TD* del = delta ? delta + (size_t)s * hidden : nullptr;
  float x[NORM_CHUNKS][4];
  float sq = 0.f;
#pragma unroll
  for (int c = 0; c < NORM_CHUNKS; ++c) {
    const int i = (c * (int)blockDim.x + threadIdx.x);
    if (i < chunks) {
      load4<float>(res + 4 * i, x[c]);
      if (del) {
        // sixteen partial sums are fetched together (one round trip), then added in index order, starting from
        // zero: the branch's output first, as a product that adds its own ranges up makes it; then the residual
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
        for (int p0 = 0; p0 < n_partials; p0 += 16) {
          float d[16][4];
#pragma unroll
          for (int p = 0; p < 16; ++p) {
            if (p0 + p < n_partials) load4<TD>(del + (size_t)(p0 + p) * partial_stride + 4 * i, d[p]);
            else d[p][0] = d[p][1] = d[p][2] = d[p][3] = 0.f;
          }
#pragma unroll
          for (int p = 0; p < 16; ++p) {
            if (p0 + p < n_partials) { sum[0] += d[p][0]; sum[1] += d[p][1]; sum[2] += d[p][2]; sum[3] += d[p][3]; }
          }
        }
        x[c][0] += sum[0]; x[c][1] += sum[1]; x[c][2] += sum[2]; x[c][3] += sum[3];
        if (write_residual) store4<float>(res + 4 * i, x[c]);
      }
      sq = fmaf(x[c][0], x[c][0], sq); sq = fmaf(x[c][1], x[c][1], sq);
      sq = fmaf(x[c][2], x[c][2], sq); sq = fmaf(x[c][3], x[c][3], sq);
    }
  }
  const float total = block_sum(sq, scratch);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
  TO* dst = out + (size_t)r * hidden;
#pragma unroll
  for (int c = 0; c < NORM_CHUNKS; ++c) {
    const int i = (c * (int)blockDim.x + threadIdx.x);
    if (i < chunks) {
      float y[4];
      y[0] = (x[c][0] * inv) * w[c][0]; y[1] = (x[c][1] * inv) * w[c][1];
      y[2] = (x[c][2] * inv) * w[c][2]; y[3] = (x[c][3] * inv) * w[c][3];
      store4<TO>(dst + 4 * i, y);
    }
  }
  LSE_TL_MARK(3)
}

// Any width: two passes over the row.
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int n_partials,
                                   long long partial_stride, const float* __restrict__ weight,
                                   TO* __restrict__ out, const int* __restrict__ rows, int hidden, float eps,
                                   int write_residual, int source_rows) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const int s = rows ? LSE_CHECKED(rows[r], -1, source_rows, -1, LSE_CHECK_ROW) : r;
  if (s < 0) return;
  float* res = residual + (size_t)s * hidden;
  const TD* del = delta ? delta + (size_t)s * hidden : nullptr;
  TO* dst = out + (size_t)r * hidden;
  float sq = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float x = res[i];
    if (del) {   // the branch's output first (its partial sums in index order, starting from zero), then the residual
      float sum = 0.f;
      for (int p = 0; p < n_partials; ++p) sum += to_f32<TD>(del[(size_t)p * partial_stride + i]);
      x += sum;
    }
    if (del && write_residual) res[i] = x;
    sq = fmaf(x, x, sq);
  }
  const float total = block_sum(sq, scratch);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float x = res[i];
    if (del && !write_residual) {
      float sum = 0.f;
      for (int p = 0; p < n_partials; ++p) sum += to_f32<TD>(del[(size_t)p * partial_stride + i]);
      x += sum;
    }
    dst[i] = from_f32<TO>((x * inv) * weight[i]);
  }
}

// Many rows (portions of prompts), one set of sums, bfloat16 out: a warp owns a row and keeps it in
// registers (C float4 chunks per lane), so that no block-wide barrier stands between the loads and
// the stores.  The norm's weights are read when they are used (they stay in the L1), which keeps the
// kernel at two blocks of eight rows an SM: 2,048 rows are all in flight at once on 148 SMs.
// hidden % 4 == 0, hidden <= 128 * C.
template <typename TD, int C>
__global__ void __launch_bounds__(256, C <= 12 ? 2 : 1)
add_rmsnorm_rows_kernel(float* __restrict__ residual, const TD* __restrict__ delta, const float* __restrict__ weight,
                        __nv_bfloat16* __restrict__ out, int n_rows, int hidden, float eps) {
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int chunks = hidden >> 2;
  pdl_wait();
  if (r >= n_rows) return;
  float* res = residual + (size_t)r * hidden;
  const TD* del = delta + (size_t)r * hidden;
  float x[C][4], d[C][4];
#pragma unroll
  for (int c = 0; c < C; ++c) {
    const int i = c * 32 + lane;
    if (i < chunks) {
      load4<float>(res + 4 * i, x[c]);
      load4<TD>(del + 4 * i, d[c]);
    }
  }
  float sq = 0.f;
#pragma unroll
  for (int c = 0; c < C; ++c) {
    const int i = c * 32 + lane;
    if (i < chunks) {
      x[c][0] += d[c][0]; x[c][1] += d[c][1]; x[c][2] += d[c][2]; x[c][3] += d[c][3];
      store4<float>(res + 4 * i, x[c]);
      sq = fmaf(x[c][0], x[c][0], sq); sq = fmaf(x[c][1], x[c][1], sq);
      sq = fmaf(x[c][2], x[c][2], sq); sq = fmaf(x[c][3], x[c][3], sq);
    }
  }
  const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)hidden + eps);
  __nv_bfloat16* dst = out + (size_t)r * hidden;
#pragma unroll
  for (int c = 0; c < C; ++c) {
    const int i = c * 32 + lane;
    if (i < chunks) {
      float w[4], y[4];
      load4<float>(weight + 4 * i, w);
      y[0] = (x[c][0] * inv) * w[0]; y[1] = (x[c][1] * inv) * w[1];
      y[2] = (x[c][2] * inv) * w[2]; y[3] = (x[c][3] * inv) * w[3];
      store4<__nv_bfloat16>(dst + 4 * i, y);
    }
  }
}

template <typename TD, typename TO>
static void launch_add_rmsnorm(float* residual, const void* delta, int n_partials, long long partial_stride,
                               const float* weight, void* out, const int* rows, int n_rows, int hidden, float eps,
                               int write_residual, int source_rows, cudaStream_t stream) {
  const bool aligned = (((uintptr_t)residual | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out) & 15) == 0 &&
                       (partial_stride % 4) == 0;
  if (sizeof(TO) == 2 && n_rows >= 256 && n_partials == 1 && delta != nullptr && rows == nullptr && write_residual &&
      hidden % 4 == 0 && hidden <= 2048 && aligned) {
    const unsigned blocks = (unsigned)((n_rows + 7) / 8);
#define LSE_NORM_ROWS(C)                                                                                        \
  lse_launch(add_rmsnorm_rows_kernel<TD, C>, blocks, 256, 0, stream, residual, (const TD*)delta, weight,        \
             (__nv_bfloat16*)out, n_rows, hidden, eps)
    if (hidden <= 512) LSE_NORM_ROWS(4);
    else if (hidden <= 1024) LSE_NORM_ROWS(8);
    else if (hidden <= 1536) LSE_NORM_ROWS(12);
    else LSE_NORM_ROWS(16);
#undef LSE_NORM_ROWS
  } else if (hidden % 4 == 0 && hidden <= NORM_THREADS * NORM_CHUNKS * 4 && aligned) {
    // few rows (decoding): one float4 chunk per thread, the shortest chain; many rows (prompts): up to
    // four chunks per thread, so that more rows are in flight on an SM
    const int per_thread = n_rows >= 256 ? NORM_CHUNKS : 1;
    int threads = (((hidden / 4 + per_thread - 1) / per_thread + 31) / 32) * 32;
    if (threads > NORM_THREADS) threads = NORM_THREADS;
    lse_launch(add_rmsnorm_vec_kernel<TD, TO>, n_rows, threads, 0, stream,
        residual, (const TD*)delta, n_partials, partial_stride, weight, (TO*)out, rows, hidden, eps, write_residual,
        source_rows);
  } else {
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    lse_launch(add_rmsnorm_kernel<TD, TO>, n_rows, threads, 0, stream,
        residual, (const TD*)delta, n_partials, partial_stride, weight, (TO*)out, rows, hidden, eps, write_residual,
        source_rows);
  }
}

extern "C" int lse_add_rmsnorm(float* residual, const void* delta, int delta_dtype, int n_partials,
                               long long partial_stride, const float* weight, void* out, int out_dtype,
                               const int* rows, int n_rows, int hidden, float eps, int write_residual,
                               int source_rows, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (delta && n_partials < 1) return LSE_ERR_BAD_ARGUMENT;
#define LSE_NORM_CASE(TD, TO)                                                                               \
  launch_add_rmsnorm<TD, TO>(residual, delta, n_partials, partial_stride, weight, out, rows, n_rows, hidden, \
                             eps, write_residual, source_rows, stream)
  if (delta_dtype == LSE_DTYPE_F32 && out_dtype == LSE_DTYPE_F32) LSE_NORM_CASE(float, float);
  else if (delta_dtype == LSE_DTYPE_BF16 && out_dtype == LSE_DTYPE_BF16) LSE_NORM_CASE(__nv_bfloat16, __nv_bfloat16);
  else if (delta_dtype == LSE_DTYPE_BF16 && out_dtype == LSE_DTYPE_F32) LSE_NORM_CASE(__nv_bfloat16, float);
  else if (delta_dtype == LSE_DTYPE_F32 && out_dtype == LSE_DTYPE_BF16) LSE_NORM_CASE(float, __nv_bfloat16);
  else return LSE_ERR_BAD_ARGUMENT;
#undef LSE_NORM_CASE
  LSE_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ rotary + bias + cache write
// qkv[t] holds the projections of token t: Hq query heads, then Hkv key heads,
// then Hkv value heads, each of D values (row stride qkv_stride; optionally a
// stack of float32 partial sums).  For every head: add the bias, rotate query
// and key heads by angle = pos * inv_freq[i] (float32), write queries to
// q_out[t, h, :] and keys/values into the paged cache at slot = slot_mapping[t]
// (page = slot / page_size, offset = slot % page_size; cache layout
// [page][kv head][offset][D]).  slot < 0: nothing is cached for this token
// (padding row).  pairing 0: pairs (2i, 2i+1); 1: (i, i+D/2).
//
// grid: (tokens, groups of heads); a thread owns four pairs of one head: eight consecutive
// elements (pairs (2i, 2i+1)) or four elements of each half (pairs (i, i + D/2)); either way the
// pairs have the frequency indices 4c .. 4c+3, c being the thread's index inside the head.
// One pair turned by its angle.  Products and sums are rounded one by one (no contraction into
// fused multiply-adds that the compiler might choose differently from kernel to kernel), so both
// kernels below give the same bits.
__device__ __forceinline__ void rope_rotate(float& xa, float& xb, float cs, float sn) {
  const float ya = __fsub_rn(__fmul_rn(xa, cs), __fmul_rn(xb, sn));
  const float yb = __fadd_rn(__fmul_rn(xb, cs), __fmul_rn(xa, sn));
  xa = ya; xb = yb;
}
template <typename T> __device__ __forceinline__ void rope_load4(const T* p, float (&v)[4]) { load4<T>(p, v); }

template <typename TI, typename TO>
__global__ void rope_kv_write_kernel(const TI* __restrict__ qkv, int n_partials, long long partial_stride,
                                     const float* __restrict__ bias, const int* __restrict__ positions,
                                     const int* __restrict__ slot_mapping, const float* __restrict__ inv_freq,
                                     TO* __restrict__ q_out, TO* __restrict__ k_cache, TO* __restrict__ v_cache,
                                     int n_q, int n_kv, int head_dim, int page_size, int pairing,
                                     long long qkv_stride, int num_slots) {
  LSE_TL_BEGIN(3)
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int per_head = head_dim >> 3;   // threads per head
  const int c = threadIdx.x % per_head;
  const int head = blockIdx.y * (blockDim.x / per_head) + threadIdx.x / per_head;   // queries, then keys, then values
  const bool in_range = head < n_q + 2 * n_kv;
  const int half = head_dim >> 1;
  // the two groups of four elements this thread owns
  const int e0 = pairing == 0 ? 8 * c : 4 * c;
  const int e1 = pairing == 0 ? 8 * c + 4 : half + 4 * c;
  const size_t col = (size_t)head * head_dim;
  // Frequencies, bias, the row's position and cache slot do not come from the kernels before this one
  // (the step's metadata is copied to the device before its first kernel starts): fetch them, and work
  // out sines and cosines, before waiting for those kernels.
  float freq[4] = {0.f, 0.f, 0.f, 0.f}, ba[4] = {0.f, 0.f, 0.f, 0.f}, bb[4] = {0.f, 0.f, 0.f, 0.f};
  float sn[4] = {0.f, 0.f, 0.f, 0.f}, cs[4] = {1.f, 1.f, 1.f, 1.f};
  int slot = -1;
  const bool is_q = head < n_q, is_k = !is_q && head < n_q + n_kv;
  if (in_range) {
    load4<float>(inv_freq + 4 * c, freq);
    if (bias) { load4<float>(bias + col + e0, ba); load4<float>(bias + col + e1, bb); }
    slot = LSE_CHECKED(slot_mapping[t], -1, num_slots, -1, LSE_CHECK_CACHE_SLOT);
    if (is_q || is_k) {
      const float pos = (float)positions[t];
#pragma unroll
      for (int j = 0; j < 4; ++j) sincosf(__fmul_rn(pos, freq[j]), &sn[j], &cs[j]);
    }
  }
  pdl_wait();
  LSE_TL_MARK(2)
  if (!in_range) return;
  if (!is_q && slot < 0) return;   // padding row: nothing is cached
  const TI* row = qkv + (size_t)t * qkv_stride + col;
  float g0[4] = {0.f, 0.f, 0.f, 0.f}, g1[4] = {0.f, 0.f, 0.f, 0.f};
  for (int p0 = 0; p0 < n_partials; p0 += 8) {   // eight partial sums per round trip, added in index order
    float a[8][4], b[8][4];
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      if (p0 + p < n_partials) {
        load4<TI>(row + (size_t)(p0 + p) * partial_stride + e0, a[p]);
        load4<TI>(row + (size_t)(p0 + p) * partial_stride + e1, b[p]);
      }
    }
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      if (p0 + p < n_partials) {
#pragma unroll
        for (int j = 0; j < 4; ++j) { g0[j] += a[p][j]; g1[j] += b[p][j]; }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) { g0[j] += ba[j]; g1[j] += bb[j]; }
  TO* dst;
  if (is_q) {
    dst = q_out + ((size_t)t * n_q + head) * head_dim;
  } else {
    const size_t page = slot / page_size, off = slot % page_size;
    const int kv_head = is_k ? head - n_q : head - n_q - n_kv;
    dst = (is_k ? k_cache : v_cache) + ((page * n_kv + kv_head) * page_size + off) * head_dim;
  }
  if (is_q || is_k) {
    float xa[4], xb[4];
    if (pairing == 0) { xa[0] = g0[0]; xb[0] = g0[1]; xa[1] = g0[2]; xb[1] = g0[3]; xa[2] = g1[0]; xb[2] = g1[1]; xa[3] = g1[2]; xb[3] = g1[3]; }
    else {
#pragma unroll
      for (int j = 0; j < 4; ++j) { xa[j] = g0[j]; xb[j] = g1[j]; }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) rope_rotate(xa[j], xb[j], cs[j], sn[j]);
    if (pairing == 0) { g0[0] = xa[0]; g0[1] = xb[0]; g0[2] = xa[1]; g0[3] = xb[1]; g1[0] = xa[2]; g1[1] = xb[2]; g1[2] = xa[3]; g1[3] = xb[3]; }
    else {
#pragma unroll
      for (int j = 0; j < 4; ++j) { g0[j] = xa[j]; g1[j] = xb[j]; }
    }
  }
  store4<TO>(dst + e0, g0);
  store4<TO>(dst + e1, g1);
  LSE_TL_MARK(3)
}

// Many tokens (256 and more: portions of prompts), one set of sums: a thread owns eight pairs (frequency indices
// 8c .. 8c+7) of ROPE_WIDE_HEADS heads of one token, so that the sines and cosines are worked out
// once for those heads and sixteen-byte loads of all of them are in flight together.  The values
// are those of the kernel above: the same angle, the same products.
constexpr int ROPE_WIDE_HEADS = 4;
template <typename T> __device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[e]);
    v[2 * e] = __low2float(h); v[2 * e + 1] = __high2float(h);
  }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float (&v)[8]);
template <> __device__ __forceinline__ void store8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
    w[e] = *reinterpret_cast<const uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

template <typename TI, typename TO>
__global__ void rope_kv_write_wide_kernel(const TI* __restrict__ qkv, const float* __restrict__ bias,
                                          const int* __restrict__ positions, const int* __restrict__ slot_mapping,
                                          const float* __restrict__ inv_freq, TO* __restrict__ q_out,
                                          TO* __restrict__ k_cache, TO* __restrict__ v_cache, int tokens, int n_q,
                                          int n_kv, int head_dim, int page_size, int pairing, long long qkv_stride,
                                          int head_groups, int num_slots) {
  pdl_launch_dependents();
  const int per_head = head_dim >> 4;            // threads per head
  const int per_token = per_head * head_groups;  // threads per token
  const int local = threadIdx.x % per_token;
  const int t = blockIdx.x * (blockDim.x / per_token) + threadIdx.x / per_token;
  const int c = local % per_head, group = local / per_head;
  const int heads = n_q + 2 * n_kv;
  const bool live = t < tokens && threadIdx.x < (blockDim.x / per_token) * per_token;
  const int e0 = pairing == 0 ? 16 * c : 8 * c;
  const int e1 = pairing == 0 ? 16 * c + 8 : (head_dim >> 1) + 8 * c;
  // position, cache slot and frequencies are the step's own data: fetched before waiting for the
  // kernel that makes the projections; the sines and cosines are worked out while the loads of the
  // projections are in flight
  float freq[8];
  int slot = -1;
  float pos = 0.f;
  if (live) {
    load8<float>(inv_freq + 8 * c, freq);
    slot = LSE_CHECKED(slot_mapping[t], -1, num_slots, -1, LSE_CHECK_CACHE_SLOT);
    pos = (float)positions[t];
  }
  pdl_wait();
  if (!live) return;
  const TI* row = qkv + (size_t)t * qkv_stride;
  float a[ROPE_WIDE_HEADS][8], b[ROPE_WIDE_HEADS][8];
#pragma unroll
  for (int k = 0; k < ROPE_WIDE_HEADS; ++k) {
    const int head = group + k * head_groups;   // neighbouring threads read neighbouring heads
    if (head < heads && (head < n_q || slot >= 0)) {
      load8<TI>(row + (size_t)head * head_dim + e0, a[k]);
      load8<TI>(row + (size_t)head * head_dim + e1, b[k]);
    }
  }
  float sn[8], cs[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) sincosf(__fmul_rn(pos, freq[j]), &sn[j], &cs[j]);
#pragma unroll
  for (int k = 0; k < ROPE_WIDE_HEADS; ++k) {
    const int head = group + k * head_groups;
    const bool is_q = head < n_q, is_k = !is_q && head < n_q + n_kv;
    if (head >= heads || (!is_q && slot < 0)) continue;   // padding row: nothing is cached
    float g0[8], g1[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { g0[j] = 0.f + a[k][j]; g1[j] = 0.f + b[k][j]; }
    if (bias) {
      float ba[8], bb[8];
      load8<float>(bias + (size_t)head * head_dim + e0, ba);
      load8<float>(bias + (size_t)head * head_dim + e1, bb);
#pragma unroll
      for (int j = 0; j < 8; ++j) { g0[j] += ba[j]; g1[j] += bb[j]; }
    }
    if (is_q || is_k) {
      if (pairing == 0) {   // pairs (2i, 2i+1): pair j of this thread lies in g0 (j < 4) or g1
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          rope_rotate(g0[2 * j], g0[2 * j + 1], cs[j], sn[j]);
          rope_rotate(g1[2 * j], g1[2 * j + 1], cs[4 + j], sn[4 + j]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) rope_rotate(g0[j], g1[j], cs[j], sn[j]);
      }
    }
    TO* dst;
    if (is_q) {
      dst = q_out + ((size_t)t * n_q + head) * head_dim;
    } else {
      const size_t page = slot / page_size, off = slot % page_size;
      const int kv_head = is_k ? head - n_q : head - n_q - n_kv;
      dst = (is_k ? k_cache : v_cache) + ((page * n_kv + kv_head) * page_size + off) * head_dim;
    }
    store8<TO>(dst + e0, g0);
    store8<TO>(dst + e1, g1);
  }
}

extern "C" int lse_rope_kv_write(const void* qkv, int in_dtype, int n_partials, long long partial_stride,
                                 const float* bias, const int* positions, const int* slot_mapping,
                                 const float* inv_freq, void* q_out, void* k_cache, void* v_cache, int out_dtype,
                                 int tokens, int n_q, int n_kv, int head_dim, int page_size, int pairing,
                                 long long qkv_stride, int num_pages, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int num_slots = num_pages * page_size;   // checked builds compare every cache slot with it
  // eight elements per thread: the head size is a multiple of 8 (16 for the half-split pairing)
  if (head_dim % 8 || (pairing == 1 && head_dim % 16) || head_dim > 2048 || page_size <= 0 ||
      (pairing != 0 && pairing != 1) || n_partials < 1 || qkv_stride % 4 || partial_stride % 4 ||
      (((uintptr_t)qkv | (uintptr_t)bias | (uintptr_t)inv_freq | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15))
    return LSE_ERR_BAD_ARGUMENT;
  const int heads = n_q + 2 * n_kv;
  const int in_vec = in_dtype == LSE_DTYPE_BF16 ? 8 : 4;   // elements of a sixteen-byte load
  if (tokens >= 256 && n_partials == 1 && head_dim % 16 == 0 && head_dim <= 1024 && qkv_stride % in_vec == 0) {
    const int per_head = head_dim / 16;
    const int head_groups = (heads + ROPE_WIDE_HEADS - 1) / ROPE_WIDE_HEADS;
    const int per_token = per_head * head_groups;
    if (per_token <= 128) {
      const int threads = 128, per_block = threads / per_token;
      const unsigned blocks = (unsigned)((tokens + per_block - 1) / per_block);
#define LSE_ROPE_WIDE_CASE(TI, TO)                                                                              \
  lse_launch(rope_kv_write_wide_kernel<TI, TO>, blocks, threads, 0, stream, (const TI*)qkv, bias, positions,    \
      slot_mapping, inv_freq, (TO*)q_out, (TO*)k_cache, (TO*)v_cache, tokens, n_q, n_kv, head_dim, page_size,   \
      pairing, qkv_stride, head_groups, num_slots)
      if (in_dtype == LSE_DTYPE_F32 && out_dtype == LSE_DTYPE_F32) LSE_ROPE_WIDE_CASE(float, float);
      else if (in_dtype == LSE_DTYPE_BF16 && out_dtype == LSE_DTYPE_BF16) LSE_ROPE_WIDE_CASE(__nv_bfloat16, __nv_bfloat16);
      else if (in_dtype == LSE_DTYPE_F32 && out_dtype == LSE_DTYPE_BF16) LSE_ROPE_WIDE_CASE(float, __nv_bfloat16);
      else return LSE_ERR_BAD_ARGUMENT;
#undef LSE_ROPE_WIDE_CASE
      LSE_LAUNCH_CHECK();
    }
  }
  const int per_head = head_dim / 8;
  int per_block = (tokens >= 64 ? 256 : 64) / per_head;   // heads per block: few tokens -> more, smaller blocks
  if (per_block < 1) per_block = 1;
  if (per_block > heads) per_block = heads;
  const int threads = per_head * per_block;
  dim3 grid(tokens, (heads + per_block - 1) / per_block);
#define LSE_ROPE_CASE(TI, TO)                                                                                   \
  lse_launch(rope_kv_write_kernel<TI, TO>, grid, threads, 0, stream,                                            \
      (const TI*)qkv, n_partials, partial_stride, bias, positions, slot_mapping, inv_freq, (TO*)q_out,          \
      (TO*)k_cache, (TO*)v_cache, n_q, n_kv, head_dim, page_size, pairing, qkv_stride, num_slots)
  if (in_dtype == LSE_DTYPE_F32 && out_dtype == LSE_DTYPE_F32) LSE_ROPE_CASE(float, float);
  else if (in_dtype == LSE_DTYPE_BF16 && out_dtype == LSE_DTYPE_BF16) LSE_ROPE_CASE(__nv_bfloat16, __nv_bfloat16);
  else if (in_dtype == LSE_DTYPE_F32 && out_dtype == LSE_DTYPE_BF16) LSE_ROPE_CASE(float, __nv_bfloat16);
  else return LSE_ERR_BAD_ARGUMENT;
#undef LSE_ROPE_CASE
  LSE_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ SiLU gate
// gate_up[t] = [gate (I values) | up (I values)];  out[t, i] = silu(gate_i) * up_i
// grid: (chunks of the row, tokens); a thread handles 4 consecutive i when I % 4 == 0.
template <typename TI, typename TO, int VEC>
__global__ void silu_mul_kernel(const TI* __restrict__ gate_up, int n_partials, long long partial_stride,
                                TO* __restrict__ out, int inter) {
  LSE_TL_BEGIN(4)
  pdl_launch_dependents();
  pdl_wait();
  LSE_TL_MARK(2)
  const int t = blockIdx.y;
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (i >= inter) return;
  const TI* row = gate_up + (size_t)t * 2 * inter;
  const int gi = i, ui = inter + i;
  float g[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f};
  for (int p = 0; p < n_partials; ++p) {
    if (VEC == 4) {
      float a[4], b[4];
      load4<TI>(row + (size_t)p * partial_stride + gi, a);
      load4<TI>(row + (size_t)p * partial_stride + ui, b);
#pragma unroll
      for (int e = 0; e < 4; ++e) { g[e] += a[e]; u[e] += b[e]; }
    } else {
      g[0] += to_f32<TI>(row[(size_t)p * partial_stride + gi]);
      u[0] += to_f32<TI>(row[(size_t)p * partial_stride + ui]);
    }
  }
  float y[4];
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    // a bfloat16 result is rounded far more coarsely than the fast exponential and division err
    if (sizeof(TO) == 2) y[e] = __fdividef(g[e], 1.0f + __expf(-g[e])) * u[e];
    else y[e] = (g[e] / (1.0f + expf(-g[e]))) * u[e];
  }
  TO* dst = out + (size_t)t * inter + i;
  if (VEC == 4) store4<TO>(dst, y);
  else dst[0] = from_f32<TO>(y[0]);
  LSE_TL_MARK(3)
}

// bfloat16 in and out, one split, I % 8 == 0: sixteen bytes per load, one load of gate and of up in
// flight per thread (more did not help: the exponentials bound it); the chunks of all rows are
// numbered flat so that no block is half empty
constexpr int SILU_UNROLL = 1;
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out,
                                       int inter, long long total_chunks) {
  LSE_TL_BEGIN(4)
  pdl_launch_dependents();
  pdl_wait();
  LSE_TL_MARK(2)
  const int per_row = inter >> 3;
  const long long first = (long long)blockIdx.x * blockDim.x * SILU_UNROLL + threadIdx.x;
  uint4 g[SILU_UNROLL], u[SILU_UNROLL];
  long long where[SILU_UNROLL];
#pragma unroll
  for (int k = 0; k < SILU_UNROLL; ++k) {
    const long long id = first + (long long)k * blockDim.x;
    where[k] = -1;
    if (id < total_chunks) {
      const long long t = id / per_row;
      const int i = (int)(id - t * per_row) * 8;
      const __nv_bfloat16* row = gate_up + t * 2 * inter;
      g[k] = *reinterpret_cast<const uint4*>(row + i);
      u[k] = *reinterpret_cast<const uint4*>(row + inter + i);
      where[k] = t * inter + i;
    }
  }
#pragma unroll
  for (int k = 0; k < SILU_UNROLL; ++k) {
    if (where[k] < 0) continue;
    const uint32_t gw[4] = {g[k].x, g[k].y, g[k].z, g[k].w}, uw[4] = {u[k].x, u[k].y, u[k].z, u[k].w};
    uint32_t yw[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __nv_bfloat162 g2 = *reinterpret_cast<const __nv_bfloat162*>(&gw[e]);
      const __nv_bfloat162 u2 = *reinterpret_cast<const __nv_bfloat162*>(&uw[e]);
      const float ga = __low2float(g2), gb = __high2float(g2);
      // the result is rounded to bfloat16: the fast exponential and division are far below that
      __nv_bfloat162 y = __floats2bfloat162_rn(__fdividef(ga, 1.0f + __expf(-ga)) * __low2float(u2),
                                               __fdividef(gb, 1.0f + __expf(-gb)) * __high2float(u2));
      yw[e] = *reinterpret_cast<uint32_t*>(&y);
    }
    *reinterpret_cast<uint4*>(out + where[k]) = make_uint4(yw[0], yw[1], yw[2], yw[3]);
  }
  LSE_TL_MARK(3)
}

extern "C" int lse_silu_mul(const void* gate_up, int in_dtype, int n_partials, long long partial_stride, void* out,
                            int out_dtype, int tokens, int inter, cudaStream_t stream) {
  if (tokens <= 0 || inter <= 0) return 0;
  if (n_partials < 1) return LSE_ERR_BAD_ARGUMENT;
  const bool vec = inter % 4 == 0 && partial_stride % 4 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0;
  const int threads = 256;
  if (vec && inter % 8 == 0 && n_partials == 1 && in_dtype == LSE_DTYPE_BF16 && out_dtype == LSE_DTYPE_BF16) {
    const long long total_chunks = (long long)tokens * (inter / 8);
    const unsigned blocks = (unsigned)((total_chunks + threads * SILU_UNROLL - 1) / (threads * SILU_UNROLL));
    lse_launch(silu_mul_bf16x8_kernel, blocks, threads, 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out,
               inter, total_chunks);
    LSE_LAUNCH_CHECK();
  }
  const int per_row = vec ? inter / 4 : inter;
  dim3 grid((per_row + threads - 1) / threads, tokens);
#define LSE_SILU_CASE(TI, TO)                                                                                      \
  if (vec) lse_launch(silu_mul_kernel<TI, TO, 4>, grid, threads, 0, stream, (const TI*)gate_up, n_partials,         \
                      partial_stride, (TO*)out, inter);                                                            \
  else lse_launch(silu_mul_kernel<TI, TO, 1>, grid, threads, 0, stream, (const TI*)gate_up, n_partials,             \
                  partial_stride, (TO*)out, inter)
  if (in_dtype == LSE_DTYPE_F32 && out_dtype == LSE_DTYPE_F32) { LSE_SILU_CASE(float, float); }
  else if (in_dtype == LSE_DTYPE_BF16 && out_dtype == LSE_DTYPE_BF16) { LSE_SILU_CASE(__nv_bfloat16, __nv_bfloat16); }
  else if (in_dtype == LSE_DTYPE_F32 && out_dtype == LSE_DTYPE_BF16) { LSE_SILU_CASE(float, __nv_bfloat16); }
  else return LSE_ERR_BAD_ARGUMENT;
#undef LSE_SILU_CASE
  LSE_LAUNCH_CHECK();
}

// Switch programmatic dependent launch on (1, the default) or off (0) for every later launch.
extern "C" int lse_set_pdl(int enabled) {
  lse_pdl_enabled = enabled ? 1 : 0;
  return 0;
}
