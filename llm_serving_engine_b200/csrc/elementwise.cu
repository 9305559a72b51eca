// Row-wise kernels of the decoder: embedding gather, RMSNorm fused with the
// residual sum, rotary position encoding fused with the bias and the write into
// the paged cache, and the SiLU gate.  Formulas follow the reference project's
// src/llmserve/model.py (RMSNorm :20-23, rotary :29-43, MLP :188).
#include "common.cuh"

// ------------------------------------------------------------------ embedding
// residual[t, :] = float(table[ids[t], :])
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ out, int hidden, int vocab) {
  const int t = blockIdx.x;
  const int id = ids[t];
  float* dst = out + (size_t)t * hidden;
  if (id < 0 || id >= vocab) {  // padding row of a fixed-shape batch
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.f;
    return;
  }
  const T* src = table + (size_t)id * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32<T>(src[i]);
}

extern "C" int lse_embedding(const void* table, int table_dtype, const int* ids, float* out,
                             int tokens, int hidden, int vocab, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (table_dtype == LSE_DTYPE_F32)
    embedding_kernel<float><<<tokens, threads, 0, stream>>>((const float*)table, ids, out, hidden, vocab);
  else if (table_dtype == LSE_DTYPE_BF16)
    embedding_kernel<__nv_bfloat16><<<tokens, threads, 0, stream>>>((const __nv_bfloat16*)table, ids, out, hidden, vocab);
  else
    return LSE_ERR_BAD_ARGUMENT;
  LSE_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ add + RMSNorm
// For output row r (source row s = rows ? rows[r] : r):
//   x = residual[s] + float(delta[s])          (delta may be null)
//   if write_residual: residual[s] = x         (float32 residual stream)
//   out[r] = (x * rsqrt(mean(x^2) + eps)) * weight
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                   const float* __restrict__ weight, TO* __restrict__ out,
                                   const int* __restrict__ rows, int hidden, float eps,
                                   int write_residual) {
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const int s = rows ? rows[r] : r;
  if (s < 0) return;
  float* res = residual + (size_t)s * hidden;
  const TD* del = delta ? delta + (size_t)s * hidden : nullptr;
  TO* dst = out + (size_t)r * hidden;
  float sq = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float x = res[i];
    if (del) x += to_f32<TD>(del[i]);
    if (del && write_residual) res[i] = x;
    sq = fmaf(x, x, sq);
  }
  const float total = block_sum(sq, scratch);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float x;
    if (del && !write_residual) x = res[i] + to_f32<TD>(del[i]);
    else x = res[i];
    dst[i] = from_f32<TO>((x * inv) * weight[i]);
  }
}

extern "C" int lse_add_rmsnorm(float* residual, const void* delta, int delta_dtype, const float* weight,
                               void* out, int out_dtype, const int* rows, int n_rows, int hidden,
                               float eps, int write_residual, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
#define LSE_NORM_CASE(TD, TO)                                                                     \
  add_rmsnorm_kernel<TD, TO><<<n_rows, threads, 0, stream>>>(residual, (const TD*)delta, weight,  \
                                                             (TO*)out, rows, hidden, eps, write_residual)
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
// then Hkv value heads, each of D values (row stride qkv_stride).  For every
// head: add the bias, rotate query and key heads by angle = pos * inv_freq[i]
// (float32), write queries to q_out[t, h, :] and keys/values into the paged
// cache at slot = slot_mapping[t] (page = slot / page_size, offset = slot %
// page_size; cache layout [page][kv head][offset][D]).  slot < 0: nothing is
// cached for this token (padding row).  pairing 0: pairs (2i, 2i+1); 1: (i, i+D/2).
template <typename T>
__global__ void rope_kv_write_kernel(const T* __restrict__ qkv, const float* __restrict__ bias,
                                     const int* __restrict__ positions,
                                     const int* __restrict__ slot_mapping,
                                     const float* __restrict__ inv_freq, T* __restrict__ q_out,
                                     T* __restrict__ k_cache, T* __restrict__ v_cache, int n_q,
                                     int n_kv, int head_dim, int page_size, int pairing,
                                     long long qkv_stride) {
  const int t = blockIdx.x;
  const int head = blockIdx.y;  // 0..n_q-1 queries, then keys, then values
  const int pos = positions[t];
  const int slot = slot_mapping[t];
  const T* src = qkv + (size_t)t * qkv_stride + (size_t)head * head_dim;
  const float* b = bias ? bias + (size_t)head * head_dim : nullptr;
  const bool is_q = head < n_q;
  const bool is_k = !is_q && head < n_q + n_kv;
  T* dst;
  if (is_q) {
    dst = q_out + ((size_t)t * n_q + head) * head_dim;
  } else {
    if (slot < 0) return;
    const int kv_head = is_k ? head - n_q : head - n_q - n_kv;
    const size_t page = slot / page_size, off = slot % page_size;
    T* base = is_k ? k_cache : v_cache;
    dst = base + ((page * n_kv + kv_head) * page_size + off) * head_dim;
  }
  if (is_q || is_k) {
    const int half = head_dim >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const int ia = pairing == 0 ? 2 * i : i;
      const int ib = pairing == 0 ? 2 * i + 1 : i + half;
      float xa = to_f32<T>(src[ia]), xb = to_f32<T>(src[ib]);
      if (b) { xa += b[ia]; xb += b[ib]; }
      const float angle = (float)pos * inv_freq[i];
      float sn, cs;
      sincosf(angle, &sn, &cs);
      dst[ia] = from_f32<T>(xa * cs - xb * sn);
      dst[ib] = from_f32<T>(xb * cs + xa * sn);
    }
  } else {
    for (int i = threadIdx.x; i < head_dim; i += blockDim.x) {
      float x = to_f32<T>(src[i]);
      if (b) x += b[i];
      dst[i] = from_f32<T>(x);
    }
  }
}

extern "C" int lse_rope_kv_write(const void* qkv, int dtype, const float* bias, const int* positions,
                                 const int* slot_mapping, const float* inv_freq, void* q_out,
                                 void* k_cache, void* v_cache, int tokens, int n_q, int n_kv,
                                 int head_dim, int page_size, int pairing, long long qkv_stride,
                                 cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (head_dim % 2 || page_size <= 0 || (pairing != 0 && pairing != 1)) return LSE_ERR_BAD_ARGUMENT;
  dim3 grid(tokens, n_q + 2 * n_kv);
  const int threads = head_dim >= 128 ? 64 : 32;
  if (dtype == LSE_DTYPE_F32)
    rope_kv_write_kernel<float><<<grid, threads, 0, stream>>>(
        (const float*)qkv, bias, positions, slot_mapping, inv_freq, (float*)q_out, (float*)k_cache,
        (float*)v_cache, n_q, n_kv, head_dim, page_size, pairing, qkv_stride);
  else if (dtype == LSE_DTYPE_BF16)
    rope_kv_write_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(
        (const __nv_bfloat16*)qkv, bias, positions, slot_mapping, inv_freq, (__nv_bfloat16*)q_out,
        (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, n_q, n_kv, head_dim, page_size, pairing,
        qkv_stride);
  else
    return LSE_ERR_BAD_ARGUMENT;
  LSE_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ SiLU gate
// gate_up[t] = [gate (I values) | up (I values)];  out[t, i] = silu(gate_i) * up_i
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter,
                                long long total) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long t = idx / inter;
  const int i = (int)(idx - t * inter);
  const float g = to_f32<T>(gate_up[t * 2 * inter + i]);
  const float u = to_f32<T>(gate_up[t * 2 * inter + inter + i]);
  const float s = g / (1.0f + expf(-g));
  out[idx] = from_f32<T>(s * u);
}

extern "C" int lse_silu_mul(const void* gate_up, void* out, int dtype, int tokens, int inter,
                            cudaStream_t stream) {
  const long long total = (long long)tokens * inter;
  if (total <= 0) return 0;
  const int threads = 256;
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  if (dtype == LSE_DTYPE_F32)
    silu_mul_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, inter, total);
  else if (dtype == LSE_DTYPE_BF16)
    silu_mul_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total);
  else
    return LSE_ERR_BAD_ARGUMENT;
  LSE_LAUNCH_CHECK();
}
