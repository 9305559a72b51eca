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

constexpr int RADIX_BITS = 11;   // the bits of a value are decided 11, 11 and 10 at a time: a histogram of 2,048 bins

// top-p: the smallest threshold t (as the bits of a float in [0, 1]) such that the mass of the values strictly greater
// than t is below top_p times the whole mass; tokens with e >= t are kept.  Found by three passes over the row, each a
// histogram of mass by the next bits of the values that share the bits decided so far (what thirty passes of a
// bisection over the float's bits gave before).  Mass is counted in integers, 2^-31 of the whole mass `total` each
// (32-bit sums, which do not depend on the order in which threads add: the threshold is the same in every run).
// top_p = 0 keeps the largest values only.
__device__ float top_p_threshold(const float* __restrict__ e, int vocab, float top_p, float total, unsigned* hist, int* chosen) {
  const float unit = 2147483648.0f / total;
  unsigned prefix = 0;              // the bits decided so far
  int done = 0;
  unsigned long long above = 0;     // mass of the values greater than every value with this prefix
  unsigned long long limit = 0;
  __shared__ unsigned long long above_s, limit_s;
  for (int level = 0; level < 3; ++level) {
    const int bits = level < 2 ? RADIX_BITS : 32 - 2 * RADIX_BITS;
    const int shift = 32 - done - bits;
    for (int b = threadIdx.x; b < (1 << bits); b += blockDim.x) hist[b] = 0;
    __syncthreads();
    // A thread adds up the values that fall into the same bin one after the other before it touches the histogram: a
    // narrow distribution (all values in a few bins) then costs an addition a thread, not one a value.  Values are
    // fetched eight at a time (two 16-byte loads in flight), neighbours in the vocabulary.
    {
      unsigned held_bin = 0xffffffffu, held = 0;
      auto take = [&](float v) {
        const unsigned u = __float_as_uint(v);
        if (done != 0 && (u >> (32 - done)) != prefix) return;
        const unsigned bin = (u >> shift) & ((1u << bits) - 1u);
        if (bin != held_bin) {
          if (held_bin != 0xffffffffu) atomicAdd(&hist[held_bin], held);
          held_bin = bin;
          held = 0;
        }
        held += __float2uint_rz(v * unit);
      };
      const int quads = (((uintptr_t)e & 15) == 0) ? vocab / 4 : 0;
      const float4* e4 = reinterpret_cast<const float4*>(e);
      for (int j = threadIdx.x; j < quads; j += 2 * blockDim.x) {
        const bool two = j + (int)blockDim.x < quads;
        const float4 a = e4[j];
        const float4 b = two ? e4[j + blockDim.x] : a;
        take(a.x); take(a.y); take(a.z); take(a.w);
        if (two) { take(b.x); take(b.y); take(b.z); take(b.w); }
      }
      for (int i = 4 * quads + threadIdx.x; i < vocab; i += blockDim.x) take(e[i]);
      if (held_bin != 0xffffffffu) atomicAdd(&hist[held_bin], held);
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      // The lowest bin whose values all leave less than `limit` above them.  A lane owns a run of bins; the mass above
      // a lane's top bin is a suffix sum over the lanes; the lowest lane whose top bin qualifies holds the bin.
      const int lane = threadIdx.x, per = (1 << bits) / 32;
      unsigned long long mine = 0;
      for (int k = 0; k < per; ++k) mine += hist[lane * per + k];
      auto shuffle_down = [](unsigned long long v, int o) {
        const unsigned lo = __shfl_down_sync(0xffffffffu, (unsigned)v, o), hi = __shfl_down_sync(0xffffffffu, (unsigned)(v >> 32), o);
        return ((unsigned long long)hi << 32) | lo;
      };
      unsigned long long suffix = mine;   // mass of this lane's bins and of all lanes above
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long v = shuffle_down(suffix, o);
        if (lane + o < 32) suffix += v;
      }
      if (level == 0) {
        const unsigned lo = __shfl_sync(0xffffffffu, (unsigned)suffix, 0), hi = __shfl_sync(0xffffffffu, (unsigned)(suffix >> 32), 0);
        limit = (unsigned long long)((double)top_p * (double)(((unsigned long long)hi << 32) | lo));
      }
      const unsigned long long over_top = above + suffix - mine;   // mass above this lane's top bin
      const unsigned qualifies = __ballot_sync(0xffffffffu, over_top < limit);
      const int holder = qualifies ? __ffs(qualifies) - 1 : 31;
      if (lane == holder) {
        unsigned long long c = over_top;
        int b = lane * per + per - 1;
        const int bottom = lane * per;
        while (b > bottom && c + hist[b] < limit) { c += hist[b]; --b; }
        *chosen = b;
        above_s = c;
        limit_s = limit;
      }
    }
    __syncthreads();
    prefix = (prefix << bits) | (unsigned)*chosen;
    above = above_s;
    limit = limit_s;
    done += bits;
    __syncthreads();
  }
  return limit == 0 ? 1.0f : __uint_as_float(prefix);   // nothing may lie above: only the largest values (e = 1) stay
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
              const float* __restrict__ temperature, const float* __restrict__ top_p,
              const long long* __restrict__ seed, const long long* __restrict__ counter,
              float* __restrict__ scratch, int* __restrict__ out) {
  __shared__ float red[32];
  __shared__ float chunk_sum[THREADS];
  __shared__ unsigned hist[1 << RADIX_BITS];
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
  // sixteen-byte loads, two of them in flight a thread, where the row allows it; the rest one value at a time
  const int quads = ((((uintptr_t)row | (uintptr_t)e) & 15) == 0) ? vocab / 4 : 0;
  const float4* row4 = reinterpret_cast<const float4*>(row);
  float4* e4 = reinterpret_cast<float4*>(e);
  float mx = -INFINITY;
  for (int j = threadIdx.x; j < quads; j += 2 * blockDim.x) {
    const float4 a = row4[j];
    const float4 b = j + (int)blockDim.x < quads ? row4[j + blockDim.x] : a;
    mx = fmaxf(mx, fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)) * inv_t);
    mx = fmaxf(mx, fmaxf(fmaxf(b.x, b.y), fmaxf(b.z, b.w)) * inv_t);
  }
  for (int i = 4 * quads + threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, row[i] * inv_t);
  mx = block_max(mx, red);
  float mass = 0.f;
  for (int j = threadIdx.x; j < quads; j += 2 * blockDim.x) {
    const bool two = j + (int)blockDim.x < quads;
    const float4 a = row4[j];
    const float4 b = two ? row4[j + blockDim.x] : a;
    const float4 ea = make_float4(expf(a.x * inv_t - mx), expf(a.y * inv_t - mx), expf(a.z * inv_t - mx), expf(a.w * inv_t - mx));
    e4[j] = ea;
    mass += (ea.x + ea.y) + (ea.z + ea.w);
    if (two) {
      const float4 eb = make_float4(expf(b.x * inv_t - mx), expf(b.y * inv_t - mx), expf(b.z * inv_t - mx), expf(b.w * inv_t - mx));
      e4[j + blockDim.x] = eb;
      mass += (eb.x + eb.y) + (eb.z + eb.w);
    }
  }
  for (int i = 4 * quads + threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = expf(row[i] * inv_t - mx);
    e[i] = v;
    mass += v;
  }
  __syncthreads();

  float keep_from = 0.f;  // keep e_i >= keep_from
  const float p = top_p[r];
  if (p < 1.0f) keep_from = top_p_threshold(e, vocab, p, block_sum(mass, red), hist, &chosen);

  // inverse CDF over the kept tokens, vocabulary order: thread c owns the chunk [c*per, (c+1)*per)
  const int per = (vocab + THREADS - 1) / THREADS;
  const int begin = min(vocab, (int)threadIdx.x * per), end = min(vocab, begin + per);
  float mine = 0.f;
  for (int i = begin; i < end; ++i) { const float v = e[i]; if (v >= keep_from) mine += v; }
  chunk_sum[threadIdx.x] = mine;
  if (threadIdx.x == 0) chosen = -1;
  __syncthreads();
  if (threadIdx.x < 32) {
    // which chunk holds the draw: a lane adds up 32 chunks, the lanes' sums are scanned, and the first lane whose
    // chunks reach the target walks them (one thread walking all 1,024 sums took 15 us)
    const int lane = threadIdx.x;
    float lane_sum = 0.f;
    for (int k = 0; k < THREADS / 32; ++k) lane_sum += chunk_sum[lane * (THREADS / 32) + k];
    float incl = lane_sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    const float total = __shfl_sync(0xffffffffu, incl, 31);
    const float target = uniform01(seed[r], counter[r]) * total;
    const unsigned reaches = __ballot_sync(0xffffffffu, incl > target);
    const int holder = reaches ? __ffs(reaches) - 1 : 31;
    if (lane != holder) return;
    float run = incl - lane_sum;     // the kept mass of the chunks before this lane's
    int c = lane * (THREADS / 32);
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
