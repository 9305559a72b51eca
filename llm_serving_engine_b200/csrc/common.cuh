// Shared device helpers for the engine's kernels (sm_100a).
//
// Conventions used by every launcher in this directory:
//   * dtype codes: 0 = float32, 1 = bfloat16.
//   * every launcher is extern "C", takes raw device pointers and the CUDA
//     stream to launch on, allocates nothing and returns a cudaError_t as int.
//   * all arithmetic inside a kernel is float32; a value is rounded once, when
//     it is stored in a bfloat16 tensor.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LSE_DTYPE_F32 0
#define LSE_DTYPE_BF16 1

// Returned (as a negative number, so that it cannot be taken for a cudaError_t)
// when a launcher refuses its arguments.
#define LSE_ERR_BAD_ARGUMENT (-1)
#define LSE_ERR_TOO_LARGE (-2)

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a whole block in a fixed order (lanes by butterfly, then warps in
// index order), so the result depends on the block size only.  `scratch` holds
// at least 32 floats.  Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < nwarps; ++w) total += scratch[w];
  return total;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = scratch[0];
  for (int w = 1; w < nwarps; ++w) total = fmaxf(total, scratch[w]);
  return total;
}

#define LSE_LAUNCH_CHECK() return (int)cudaGetLastError()

// ------------------------------------------------------------------ launches
// Every kernel of the library is launched with programmatic dependent launch allowed:
// the next kernel of the stream may be scheduled while this one still runs.  A kernel
// calls pdl_launch_dependents() when it starts and pdl_wait() before it first touches
// anything an earlier kernel of the stream wrote (and before it writes global memory at
// all); what lies before pdl_wait() (setting up barriers, fetching weights) overlaps the
// tail of the kernel before.  pdl_wait() returns when the earlier kernels have finished
// and their writes are visible; it is a no-op when the launch carried no such permission.
inline int lse_pdl_enabled = 1;

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// Which request's which rows the block of rank `rank` covers, when every request's rows (segment_start[s] ..
// segment_start[s + 1]) are cut into tiles of rows_per_tile rows (requests of one row take none when skip_single).
// Tiles are numbered request by request and handed out from the last one backwards: rank 0 takes the last tile (late
// tiles walk the most keys and should start first), and the ranks beyond the number of tiles (a grid is sized by an
// upper bound) come last and leave at once.  The block's first warp works it out, 32 requests at a time (a step may
// hold hundreds), and hands it to the other warps through `slot` (three ints of shared memory).  Every thread of
// the block calls it; it ends with a __syncthreads().  seg = -1: the rank has no tile.
__device__ __forceinline__ void lse_find_tile(const int* __restrict__ segment_start, int num_segments, int rows_per_tile,
                                              int skip_single, int rank, int* slot, int& seg, int& r0, int& cnt) {
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    auto tiles_of = [&](int s, int& c) {
      c = 0;
      if (s >= num_segments) return 0;
      c = segment_start[s + 1] - segment_start[s];
      return (skip_single && c == 1) ? 0 : (c + rows_per_tile - 1) / rows_per_tile;
    };
    int total = 0;
    for (int base = 0; base < num_segments; base += 32) {
      int c;
      int nt = tiles_of(base + lane, c);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) nt += __shfl_xor_sync(0xffffffffu, nt, o);
      total += nt;
    }
    const int tile = total - 1 - rank;
    int before = 0, found_seg = -1, found_r0 = 0, found_cnt = 0;   // the same in every lane
    for (int base = 0; base < num_segments && found_seg < 0 && tile >= 0; base += 32) {
      int c;
      const int nt = tiles_of(base + lane, c);
      int incl = nt;   // tiles of the requests base .. base + lane
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      const int excl = incl - nt;
      const unsigned vote = __ballot_sync(0xffffffffu, nt > 0 && tile >= before + excl && tile < before + incl);
      if (vote) {
        const int src = __ffs(vote) - 1;
        found_seg = base + src;
        found_r0 = (tile - before - __shfl_sync(0xffffffffu, excl, src)) * rows_per_tile;
        found_cnt = __shfl_sync(0xffffffffu, c, src);
      }
      before += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) { slot[0] = found_seg; slot[1] = found_r0; slot[2] = found_cnt; }
  }
  __syncthreads();
  seg = slot[0]; r0 = slot[1]; cnt = slot[2];
}

// cluster_z > 1: the blocks (x, y, 0 .. cluster_z-1) form a thread-block cluster (distributed shared memory).
template <typename... KArgs, typename... Args>
inline cudaError_t lse_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t stream, unsigned cluster_z, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = lse_pdl_enabled ? 1 : 0;
  config.attrs = attribute;
  config.numAttrs = 1;
  if (cluster_z > 1) {
    attribute[1].id = cudaLaunchAttributeClusterDimension;
    attribute[1].val.clusterDim.x = 1;
    attribute[1].val.clusterDim.y = 1;
    attribute[1].val.clusterDim.z = cluster_z;
    config.numAttrs = 2;
  }
  return cudaLaunchKernelEx(&config, kernel, static_cast<Args&&>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t lse_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  return lse_launch_cluster(kernel, grid, block, smem, stream, 1u, static_cast<Args&&>(args)...);
}


// ------------------------------------------------------------------ checked builds
// With -DLSE_CHECK every index that a kernel takes from the step's metadata (token ids, cache slots,
// block-table entries inside the context, segment numbers, gathered rows) is compared with its range
// before it is used.  An index out of range is replaced by a safe one, so that nothing outside the
// buffers is touched, and the first violation of each source file is recorded (what kind, the value,
// the range) for the host to read with the exported reader.  Nothing traps.  Without the flag the
// macros cost nothing: LSE_CHECKED(value, ...) is `value`.
#define LSE_CHECK_TOKEN_ID 1
#define LSE_CHECK_CACHE_SLOT 2
#define LSE_CHECK_TABLE_ENTRY 3
#define LSE_CHECK_SEGMENT 4
#define LSE_CHECK_ROW 5
#ifdef LSE_CHECK
#define LSE_CHECK_DEFINE(reader)                                                                           \
  __device__ int lse_check_word[4];                                                                        \
  extern "C" int reader(int* host_out, int reset) {                                                        \
    if (cudaMemcpyFromSymbol(host_out, lse_check_word, sizeof(int) * 4) != cudaSuccess) return -1;          \
    if (reset) { const int zero[4] = {0, 0, 0, 0}; cudaMemcpyToSymbol(lse_check_word, zero, sizeof(zero)); } \
    return 0;                                                                                              \
  }
__device__ __forceinline__ int lse_checked(int value, int lo, int hi, int safe, int kind, int* word) {
  if (value >= lo && value < hi) return value;
  if (atomicCAS(&word[0], 0, kind) == 0) { word[1] = value; word[2] = lo; word[3] = hi; }
  return safe;
}
#define LSE_CHECKED(value, lo, hi, safe, kind) lse_checked((value), (lo), (hi), (safe), (kind), lse_check_word)
#else
#define LSE_CHECK_DEFINE(reader)
#define LSE_CHECKED(value, lo, hi, safe, kind) (value)
#endif

// ------------------------------------------------------------------ timeline (tuning builds only)
// With -DLSE_TRACE every kernel's block 0 records when it started, when pdl_wait() returned and
// when it ended (nanoseconds of %globaltimer) into a per-source-file buffer that a tuning script
// reads back with the exported reader.  Without the flag the macros vanish.
#ifdef LSE_TRACE
#define LSE_TL_CAPACITY 4096
#define LSE_TL_DEFINE(reader)                                                                              \
  __device__ unsigned long long lse_tl_data[LSE_TL_CAPACITY * 8];                                          \
  __device__ unsigned int lse_tl_count;                                                                    \
  __device__ volatile int lse_tl_last = -1;                                                                \
  extern "C" int reader(unsigned long long* host_out, int reset) {                                         \
    unsigned int n = 0;                                                                                    \
    cudaMemcpyFromSymbol(&n, lse_tl_count, sizeof(n));                                                     \
    if (n > LSE_TL_CAPACITY) n = LSE_TL_CAPACITY;                                                          \
    if (n) cudaMemcpyFromSymbol(host_out, lse_tl_data, sizeof(unsigned long long) * 8 * n);                \
    if (reset) { unsigned int zero = 0; cudaMemcpyToSymbol(lse_tl_count, &zero, sizeof(zero)); }           \
    return (int)n;                                                                                         \
  }
__device__ __forceinline__ unsigned long long lse_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define LSE_TL_BEGIN(id)                                                                                   \
  int tl_slot_ = -1;                                                                                       \
  if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {                         \
    tl_slot_ = (int)atomicAdd(&lse_tl_count, 1u);                                                          \
    if (tl_slot_ < LSE_TL_CAPACITY) { lse_tl_data[tl_slot_ * 8] = (id); lse_tl_data[tl_slot_ * 8 + 1] = lse_now(); lse_tl_last = tl_slot_; } \
    else tl_slot_ = -1;                                                                                    \
  }
#define LSE_TL_MARK(k) if (tl_slot_ >= 0) lse_tl_data[tl_slot_ * 8 + (k)] = lse_now();
// a mark by some other block of the same launch (the slot of the launch's block 0 is read back)
#define LSE_TL_MARK_ANY(k, cond) if (cond) { const int sl_ = lse_tl_last; if (sl_ >= 0 && sl_ < LSE_TL_CAPACITY) lse_tl_data[sl_ * 8 + (k)] = lse_now(); }
#else
#define LSE_TL_DEFINE(reader)
#define LSE_TL_BEGIN(id)
#define LSE_TL_MARK(k)
#define LSE_TL_MARK_ANY(k, cond)
#endif
