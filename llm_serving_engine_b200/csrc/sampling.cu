// Token selection on the device: argmax, and temperature / top-p sampling by
// inverse CDF in vocabulary order with a counter-based random number.
//
// The reference samples with torch.softmax + torch.multinomial and, for
// top-p, a descending sort (src/llmserve/engine.py:29-72).  Here the same
// distribution is drawn without a sort and without a library generator:
//   z_i = logit_i / temperature;  e_i = exp(z_i - max z);  Z = sum e_i
//   top-p keeps token i when the mass of the tokens with a strictly larger e
//   is below top_p * Z (the reference's "cumulative - own >= top_p" removal,
//   engine.py:34-38; tokens that tie with the last kept one are kept too);
//   u = uniform(seed, counter) in [0, 1);  the token is the first kept i, in
//   vocabulary order, whose running kept mass exceeds u * (kept mass).
// uniform(): splitmix64 of (seed, counter), upper 24 bits.
//
// One block per row.  `scratch` holds rows * vocab floats (the e_i).
#include "common.cuh"

namespace {
constexpr int THREADS = 1024;

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
__device__ __forceinline__ float uniform01(long long seed, long long counter) {
  const unsigned long long h =
      splitmix64(splitmix64((unsigned long long)seed) ^ ((unsigned long long)counter * 0xD1342543DE82EF95ull + 1ull));
  return (float)(h >> 40) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(THREADS)
argmax_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
              int* __restrict__ out) {
  __shared__ float best_v[32];
  __shared__ int best_i[32];
  pdl_launch_dependents();
  pdl_wait();
  const float* row = logits + (size_t)blockIdx.x * row_stride;
  float bv = -INFINITY;
  int bi = vocab;  // "none yet"
  // Sixteen values per thread and round (four 16-byte loads in flight), taken in ascending order of the index, so
  // that the first maximum wins inside a thread; between threads the smaller index wins a tie (below).
  const bool vec = (vocab & 3) == 0 && (((uintptr_t)row) & 15) == 0;
  const int n4 = vec ? vocab >> 2 : 0;
  for (int c0 = threadIdx.x; c0 < n4; c0 += 4 * blockDim.x) {
    float4 v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = c0 + k * blockDim.x;
      v[k] = c < n4 ? reinterpret_cast<const float4*>(row)[c] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i = (c0 + k * (int)blockDim.x) * 4;
      if (i >= vocab) continue;
      if (v[k].x > bv || bi == vocab) { bv = v[k].x; bi = i; }
      if (v[k].y > bv) { bv = v[k].y; bi = i + 1; }
      if (v[k].z > bv) { bv = v[k].z; bi = i + 2; }
      if (v[k].w > bv) { bv = v[k].w; bi = i + 3; }
    }
  }
  for (int i = n4 * 4 + threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    if (v > bv || bi == vocab) { bv = v; bi = i; }  // ascending i per thread: first maximum wins
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) { bv = best_v[w]; bi = best_i[w]; }
    out[blockIdx.x] = bi < vocab ? bi : 0;
  }
}

// Sum of the values of `e` that are greater than `threshold`, in a fixed order.
__device__ float mass_above(const float* e, int vocab, float threshold, float* red) {
  float s = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = e[i];
    if (v > threshold) s += v;
  }
  return block_sum(s, red);
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
              const float* __restrict__ temperature, const float* __restrict__ top_p,
              const long long* __restrict__ seed, const long long* __restrict__ counter,
              float* __restrict__ scratch, int* __restrict__ out) {
  __shared__ float red[32];
  __shared__ float chunk_sum[THREADS];
  __shared__ int chosen;
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * row_stride;
  float* e = scratch + (size_t)r * vocab;
  const float temp = temperature[r];
  if (!(temp > 0.f)) {  // greedy row inside a sampled batch
    float bv = -INFINITY; int bi = vocab;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float v = row[i];
      if (v > bv || bi == vocab) { bv = v; bi = i; }
    }
    // reuse chunk_sum/red as the reduction space
    __shared__ int idx[THREADS];
    chunk_sum[threadIdx.x] = bv; idx[threadIdx.x] = bi;
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < THREADS; ++w)
        if (chunk_sum[w] > bv || (chunk_sum[w] == bv && idx[w] < bi)) { bv = chunk_sum[w]; bi = idx[w]; }
      out[r] = bi < vocab ? bi : 0;
    }
    return;
  }
  const float inv_t = 1.0f / temp;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, row[i] * inv_t);
  mx = block_max(mx, red);
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) e[i] = expf(row[i] * inv_t - mx);
  __syncthreads();

  // top-p: smallest threshold (as float bits) whose strictly-greater mass is below top_p * Z
  float keep_from = 0.f;  // keep e_i >= keep_from
  const float p = top_p[r];
  if (p < 1.0f) {
    const float total = mass_above(e, vocab, -1.f, red);
    const float limit = p * total;
    unsigned lo = 0u, hi = 0x3F800000u;  // bits of 0.0f .. 1.0f; e_i <= 1 so mass_above(1.0) = 0 < limit
    while (lo < hi) {
      const unsigned mid = lo + ((hi - lo) >> 1);
      const float m = mass_above(e, vocab, __uint_as_float(mid), red);
      if (m < limit) hi = mid; else lo = mid + 1;
    }
    keep_from = __uint_as_float(lo);
  }

  // inverse CDF over the kept tokens, vocabulary order: thread c owns the chunk [c*per, (c+1)*per)
  const int per = (vocab + THREADS - 1) / THREADS;
  const int begin = min(vocab, (int)threadIdx.x * per), end = min(vocab, begin + per);
  float mine = 0.f;
  for (int i = begin; i < end; ++i) { const float v = e[i]; if (v >= keep_from) mine += v; }
  chunk_sum[threadIdx.x] = mine;
  if (threadIdx.x == 0) chosen = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int c = 0; c < THREADS; ++c) total += chunk_sum[c];
    const float target = uniform01(seed[r], counter[r]) * total;
    float run = 0.f;
    int c = 0;
    for (; c < THREADS - 1; ++c) {
      if (run + chunk_sum[c] > target) break;
      run += chunk_sum[c];
    }
    // walk the chunk (the last chunks absorb rounding: fall back to the last kept token)
    int pick = -1, last_kept = -1;
    for (int cc = c; cc < THREADS && pick < 0; ++cc) {
      const int b = min(vocab, cc * per), en = min(vocab, b + per);
      for (int i = b; i < en; ++i) {
        const float v = e[i];
        if (v >= keep_from) {
          last_kept = i;
          run += v;
          if (run > target) { pick = i; break; }
        }
      }
    }
    if (pick < 0) {
      if (last_kept < 0)
        for (int i = vocab - 1; i >= 0; --i) if (e[i] >= keep_from) { last_kept = i; break; }
      pick = last_kept < 0 ? 0 : last_kept;
    }
    out[r] = pick;
  }
}
}  // namespace

extern "C" int lse_argmax(const float* logits, long long row_stride, int rows, int vocab, int* out,
                          cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return LSE_ERR_BAD_ARGUMENT;
  lse_launch(argmax_kernel, rows, THREADS, 0, stream, logits, row_stride, vocab, out);
  LSE_LAUNCH_CHECK();
}

extern "C" int lse_sample(const float* logits, long long row_stride, int rows, int vocab,
                          const float* temperature, const float* top_p, const long long* seed,
                          const long long* counter, float* scratch, int* out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return LSE_ERR_BAD_ARGUMENT;
  lse_launch(sample_kernel, rows, THREADS, 0, stream, logits, row_stride, vocab, temperature, top_p, seed,
             counter, scratch, out);
  LSE_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------
// lse_sample_noalloc: the same sampling kernel with scratch that lives in the library image,
// for callers that cannot allocate device memory.  See sampling_noalloc.h for the contract.
// ------------------------------------------------------------------------------------------
#include <stdio.h>

#include "sampling_noalloc.h"

// The scratch itself.  In device code this name is the array; in host code it is only a
// handle for cudaGetSymbolAddress and must never be passed to a kernel as if it were a pointer.
static __device__ __align__(256) float lse_noalloc_scratch[LSE_SAMPLE_NOALLOC_MAX_FLOATS];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
float* noalloc_scratch_of_device[NOALLOC_MAX_DEVICES];   // device address of the array, per device; null = not looked up yet
}  // namespace

extern "C" int lse_sample_noalloc(const float* logits, long long row_stride, int rows, int vocab,
                                  const float* temperature, const float* top_p, const long long* seed,
                                  const long long* counter, int* out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || !logits || !temperature || !top_p || !seed || !counter || !out)
    return LSE_SAMPLE_NOALLOC_BAD_ARGUMENT;
  if ((long long)rows * (long long)vocab > (long long)LSE_SAMPLE_NOALLOC_MAX_FLOATS) {
    fprintf(stderr,
            "lse_sample_noalloc: %d rows x %d vocabulary = %lld floats of scratch, but the built-in scratch "
            "holds %d; sample fewer rows per call or use lse_sample with your own buffer\n",
            rows, vocab, (long long)rows * vocab, (int)LSE_SAMPLE_NOALLOC_MAX_FLOATS);
    return LSE_SAMPLE_NOALLOC_TOO_LARGE;
  }
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return (int)err;
  if (device < 0 || device >= NOALLOC_MAX_DEVICES) return LSE_SAMPLE_NOALLOC_BAD_ARGUMENT;
  float* scratch = noalloc_scratch_of_device[device];
  if (scratch == nullptr) {
    // first call on this device (which is current): ask the runtime where the array lives here
    err = cudaGetSymbolAddress((void**)&scratch, lse_noalloc_scratch);
    if (err != cudaSuccess) return (int)err;
    if (scratch == nullptr) return LSE_SAMPLE_NOALLOC_BAD_ARGUMENT;
    noalloc_scratch_of_device[device] = scratch;
  }
  sample_kernel<<<rows, THREADS, 0, stream>>>(logits, row_stride, vocab, temperature, top_p, seed, counter,
                                              scratch, out);
  return (int)cudaGetLastError();
}
