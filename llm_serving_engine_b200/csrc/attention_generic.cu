// Paged attention, general form: any head size that is a multiple of 16 (up to
// 256), any number of heads and groups, any page size, float32 or bfloat16
// storage, optional window.  One block computes one query row (one token of the
// step) for up to GC query heads that share one key/value head.
//
// For row t of the step: the request's pages are block_tables[segment_of_token[t]],
// its position is positions[t], and it attends to keys j with
//     max(0, pos + 1 - window) <= j <= pos        (window <= 0: all keys j <= pos).
// Keys are walked in tiles of KT in logical order with the online-softmax
// recurrence of the reference (src/llmserve/model.py:143-176;
// src/llmserve/triton_kernels/paged_attention.py:62-138):
//     s_j = (q . k_j) * scale;  m' = max(m, max_j s_j);  c = exp(m - m')
//     p_j = exp(s_j - m');  acc = acc * c + sum_j p_j v_j;  l = l * c + sum_j p_j
//     out = acc / l
// A row's keys are summed chunk by chunk (CHUNK keys, counted from key 0): the recurrence above
// runs inside a chunk, and the chunks' (max, sum, acc) are merged in order,
//     m' = max(M, m_c);  a = exp(M - m');  b = exp(m_c - m');  A = A a + acc_c b;  L = L a + l_c b.
// With many rows one block walks all chunks of its row; with few rows (decoding) every chunk has a
// block of its own, which leaves its partial result in global memory, and a second kernel merges them
// with the same operations in the same order.  Chunks and tiles depend on the row's own position only,
// so a row's result is the same bit for bit whatever else is in the batch, however the prompt was cut
// and whichever of the two ways ran.
//
// Cache layout: [page][kv head][offset in page][D].
#include "common.cuh"

LSE_CHECK_DEFINE(lse_check_attention_generic)

namespace {
constexpr int KT = 32;        // keys per tile (one warp lane per key)
constexpr int CHUNK = 256;    // keys per chunk (a multiple of KT)
constexpr int GC = 8;         // query heads per block (chunk of a group)
constexpr int THREADS = 128;  // 4 warps
constexpr int MAX_D = 256;
constexpr int DPT = MAX_D / THREADS;  // output values per thread and head

// Merge a chunk's (m, l) into the running (M, L); wa and wb are the factors for the outputs.
__device__ __forceinline__ void merge_chunk(float& M, float& L, float m, float l, float& wa, float& wb) {
  const float m_new = fmaxf(M, m);
  wa = expf(M - m_new);    // exp(-inf) = 0 before the first chunk; every chunk of a row has a visible key, so m is finite
  wb = expf(m - m_new);
  L = fmaf(l, wb, L * wa);
  M = m_new;
}

// SPLIT: blockIdx.z also numbers the chunk; the block writes acc [D], m, l of its chunk and heads to
// `partials` [t][head][chunk][D + 2] and leaves.  Else the block merges all chunks of its row and writes `out`.
template <typename T, bool SPLIT>
__global__ void __launch_bounds__(THREADS)
paged_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_cache,
                               const T* __restrict__ v_cache, T* __restrict__ out,
                               const int* __restrict__ block_tables, int bt_stride,
                               const int* __restrict__ segment_of_token,
                               const int* __restrict__ positions, int n_q, int n_kv, int head_dim,
                               int page_size, float scale, int window, int num_pages, int num_segments,
                               float* __restrict__ partials, int max_chunks) {
  extern __shared__ float smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int kv_head = blockIdx.y;
  const int group = n_q / n_kv;
  const int gchunks = (group + GC - 1) / GC;
  const int g0 = (SPLIT ? blockIdx.z % gchunks : blockIdx.z) * GC;
  const int gcount = min(GC, group - g0);
  const int seg = LSE_CHECKED(segment_of_token[t], -1, num_segments, -1, LSE_CHECK_SEGMENT);
  if (seg < 0) return;
  const int pos = positions[t];
  const int ctx = pos + 1;
  const int kv_begin = window > 0 ? max(0, ctx - window) : 0;
  int chunk_lo = kv_begin / CHUNK, chunk_hi = pos / CHUNK;
  if (SPLIT) {
    const int mine = blockIdx.z / gchunks;
    if (mine < chunk_lo || mine > chunk_hi) return;
    chunk_lo = chunk_hi = mine;
  }
  const int* bt = block_tables + (size_t)seg * bt_stride;

  const int D = head_dim;
  float* q_s = smem;                       // [GC][D]
  float* k_s = q_s + GC * D;               // [KT][D + 1]
  float* v_s = k_s + KT * (D + 1);         // [KT][D]
  float* p_s = v_s + KT * D;               // [GC][KT]
  float* corr_s = p_s + GC * KT;           // [GC]
  float* l_s = corr_s + GC;                // [GC]
  float* m_s = l_s + GC;                   // [GC]
  long long* base_s = (long long*)(m_s + GC);  // [KT] element offset of key j in the cache, -1 = masked

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int first_head = kv_head * group + g0;
  for (int e = tid; e < gcount * D; e += THREADS) {
    const int g = e / D, d = e % D;
    q_s[g * D + d] = to_f32<T>(q[((size_t)t * n_q + first_head + g) * D + d]);
  }

  // the row's running result over its chunks (every thread keeps the maxima and sums of all heads)
  float total[GC][DPT], M[GC], L[GC];
#pragma unroll
  for (int g = 0; g < GC; ++g) {
    M[g] = -INFINITY;
    L[g] = 0.f;
#pragma unroll
    for (int i = 0; i < DPT; ++i) total[g][i] = 0.f;
  }

  for (int chunk = chunk_lo; chunk <= chunk_hi; ++chunk) {
    float acc[GC][DPT];
#pragma unroll
    for (int g = 0; g < GC; ++g)
#pragma unroll
      for (int i = 0; i < DPT; ++i) acc[g][i] = 0.f;
    // running max and sum of the heads this warp owns (g = warp, warp + 4), same value in every lane
    float m_run[GC / 4], l_run[GC / 4];
#pragma unroll
    for (int i = 0; i < GC / 4; ++i) { m_run[i] = -INFINITY; l_run[i] = 0.f; }

    const int tile_begin = max(chunk * CHUNK, (kv_begin / KT) * KT);
    const int tile_end = min(ctx, (chunk + 1) * CHUNK);
    for (int base = tile_begin; base < tile_end; base += KT) {
      __syncthreads();  // previous tile fully consumed (also orders the q_s fill)
      if (tid < KT) {
        const int j = base + tid;
        long long off = -1;
        if (j < ctx && j >= kv_begin) {
          const int page = LSE_CHECKED(bt[j / page_size], 0, num_pages, 0, LSE_CHECK_TABLE_ENTRY);
          off = (((long long)page * n_kv + kv_head) * page_size + (j % page_size)) * D;
        }
        base_s[tid] = off;
      }
      __syncthreads();
      for (int e = tid; e < KT * D; e += THREADS) {
        const int j = e / D, d = e % D;
        const long long off = base_s[j];
        float kv = 0.f, vv = 0.f;
        if (off >= 0) { kv = to_f32<T>(k_cache[off + d]); vv = to_f32<T>(v_cache[off + d]); }
        k_s[j * (D + 1) + d] = kv;
        v_s[j * D + d] = vv;
      }
      __syncthreads();
      // scores and softmax statistics: warp w owns heads g = w, w + 4; lane = key
#pragma unroll
      for (int i = 0; i < GC / 4; ++i) {
        const int g = warp + 4 * i;
        if (g < gcount) {
          const bool valid = base_s[lane] >= 0;
          float s = 0.f;
          const float* qr = q_s + g * D;
          const float* kr = k_s + lane * (D + 1);
          for (int d = 0; d < D; ++d) s = fmaf(qr[d], kr[d], s);
          s = valid ? s * scale : -INFINITY;
          const float m_new = fmaxf(m_run[i], warp_max(s));
          const float c = expf(m_run[i] - m_new);  // exp(-inf) = 0 on the first tile
          const float p = valid ? expf(s - m_new) : 0.f;
          p_s[g * KT + lane] = p;
          float tile_sum = 0.f;  // keys in order, the same in every lane
          for (int j = 0; j < KT; ++j) tile_sum += __shfl_sync(0xffffffffu, p, j);
          l_run[i] = l_run[i] * c + tile_sum;
          m_run[i] = m_new;
          if (lane == 0) { corr_s[g] = c; l_s[g] = l_run[i]; m_s[g] = m_new; }
        }
      }
      __syncthreads();
      // acc = acc * c + P V: thread owns output columns d = tid, tid + 128
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        const int d = tid + i * THREADS;
        if (d < D) {
#pragma unroll
          for (int g = 0; g < GC; ++g) {
            if (g < gcount) {
              float a = acc[g][i] * corr_s[g];
              const float* pr = p_s + g * KT;
              for (int j = 0; j < KT; ++j) a = fmaf(pr[j], v_s[j * D + d], a);
              acc[g][i] = a;
            }
          }
        }
      }
    }
    __syncthreads();   // m_s and l_s of the chunk's last tile
    if (SPLIT) {
#pragma unroll
      for (int g = 0; g < GC; ++g) {
        if (g < gcount) {
          float* dst = partials + (((size_t)t * n_q + first_head + g) * max_chunks + chunk) * (D + 2);
#pragma unroll
          for (int i = 0; i < DPT; ++i) {
            const int d = tid + i * THREADS;
            if (d < D) dst[d] = acc[g][i];
          }
          if (tid == 0) { dst[D] = m_s[g]; dst[D + 1] = l_s[g]; }
        }
      }
      return;
    }
#pragma unroll
    for (int g = 0; g < GC; ++g) {
      if (g < gcount) {
        float wa, wb;
        merge_chunk(M[g], L[g], m_s[g], l_s[g], wa, wb);
#pragma unroll
        for (int i = 0; i < DPT; ++i) total[g][i] = fmaf(acc[g][i], wb, total[g][i] * wa);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    const int d = tid + i * THREADS;
    if (d < D) {
#pragma unroll
      for (int g = 0; g < GC; ++g) {
        if (g < gcount)
          out[((size_t)t * n_q + first_head + g) * D + d] = from_f32<T>(total[g][i] / L[g]);
      }
    }
  }
}

// The chunks of a row and head, left by the SPLIT kernel, merged in order: grid (tokens, n_q), a thread per column.
template <typename T>
__global__ void __launch_bounds__(MAX_D)
paged_attention_generic_merge_kernel(const float* __restrict__ partials, T* __restrict__ out,
                                     const int* __restrict__ segment_of_token, const int* __restrict__ positions,
                                     int n_q, int head_dim, int window, int max_chunks, int num_segments) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, head = blockIdx.y, d = threadIdx.x;
  const int seg = LSE_CHECKED(segment_of_token[t], -1, num_segments, -1, LSE_CHECK_SEGMENT);
  if (seg < 0 || d >= head_dim) return;
  const int pos = positions[t];
  const int kv_begin = window > 0 ? max(0, pos + 1 - window) : 0;
  const float* src = partials + ((size_t)t * n_q + head) * max_chunks * (head_dim + 2);
  float total = 0.f, M = -INFINITY, L = 0.f;
  for (int chunk = kv_begin / CHUNK; chunk <= pos / CHUNK; ++chunk) {
    const float* part = src + (size_t)chunk * (head_dim + 2);
    float wa, wb;
    merge_chunk(M, L, part[head_dim], part[head_dim + 1], wa, wb);
    total = fmaf(part[d], wb, total * wa);
  }
  out[((size_t)t * n_q + head) * head_dim + d] = from_f32<T>(total / L);
}

size_t generic_smem_bytes(int D) {
  return sizeof(float) * ((size_t)GC * D + (size_t)KT * (D + 1) + (size_t)KT * D + GC * KT + 3 * GC) +
         sizeof(long long) * KT + 16;
}
}  // namespace

// Keys of a chunk (the caller sizes `partials` by it).
extern "C" int lse_attention_generic_chunk(void) { return CHUNK; }

// partials != null: every chunk of a row gets a block of its own (few rows: decoding) and a second
// kernel merges them; partials holds tokens * n_q * max_chunks * (head_dim + 2) floats, and max_chunks
// chunks cover the longest context that the block tables can describe.  The result is the same bit
// for bit either way.
extern "C" int lse_paged_attention_generic(const void* q, const void* k_cache, const void* v_cache,
                                           void* out, int dtype, const int* block_tables,
                                           int bt_stride, const int* segment_of_token,
                                           const int* positions, int tokens, int n_q, int n_kv,
                                           int head_dim, int page_size, float scale, int window,
                                           int num_pages, int num_segments, float* partials, int max_chunks,
                                           cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (head_dim <= 0 || head_dim > MAX_D || head_dim % 16 || n_kv <= 0 || n_q % n_kv || page_size <= 0)
    return LSE_ERR_BAD_ARGUMENT;
  const int group = n_q / n_kv;
  const int gchunks = (group + GC - 1) / GC;
  const bool split = partials != nullptr;
  if (split && (max_chunks <= 0 || (long long)gchunks * max_chunks > 65535 ||
                (long long)max_chunks * CHUNK < (long long)bt_stride * page_size))
    return LSE_ERR_BAD_ARGUMENT;
  dim3 grid(tokens, n_kv, split ? gchunks * max_chunks : gchunks);
  const size_t smem = generic_smem_bytes(head_dim);
  // the largest head size once per process (not repeated while a stream is captured)
  static bool configured = false;
  if (!configured) {
    const int most = (int)generic_smem_bytes(MAX_D);
    cudaError_t err = cudaFuncSetAttribute(paged_attention_generic_kernel<float, false>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(paged_attention_generic_kernel<float, true>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(paged_attention_generic_kernel<__nv_bfloat16, false>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(paged_attention_generic_kernel<__nv_bfloat16, true>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  const dim3 merge_grid(tokens, n_q);
  const int merge_threads = ((head_dim + 31) / 32) * 32;
#define LSE_GENERIC_CASE(T)                                                                                       \
  if (split) {                                                                                                    \
    lse_launch(paged_attention_generic_kernel<T, true>, grid, THREADS, smem, stream, (const T*)q,                 \
        (const T*)k_cache, (const T*)v_cache, (T*)out, block_tables, bt_stride, segment_of_token, positions, n_q,  \
        n_kv, head_dim, page_size, scale, window, num_pages, num_segments, partials, max_chunks);                 \
    lse_launch(paged_attention_generic_merge_kernel<T>, merge_grid, merge_threads, 0, stream,                     \
        (const float*)partials, (T*)out, segment_of_token, positions, n_q, head_dim, window, max_chunks,          \
        num_segments);                                                                                            \
  } else {                                                                                                        \
    lse_launch(paged_attention_generic_kernel<T, false>, grid, THREADS, smem, stream, (const T*)q,                \
        (const T*)k_cache, (const T*)v_cache, (T*)out, block_tables, bt_stride, segment_of_token, positions, n_q,  \
        n_kv, head_dim, page_size, scale, window, num_pages, num_segments, (float*)nullptr, 0);                   \
  }
  if (dtype == LSE_DTYPE_F32) { LSE_GENERIC_CASE(float) }
  else if (dtype == LSE_DTYPE_BF16) { LSE_GENERIC_CASE(__nv_bfloat16) }
  else return LSE_ERR_BAD_ARGUMENT;
#undef LSE_GENERIC_CASE
  LSE_LAUNCH_CHECK();
}
