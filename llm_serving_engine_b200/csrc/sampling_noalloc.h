/* lse_sample_noalloc: token sampling for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference project (Arnavsharma2/llm-serving-engine
 * samples with torch ops, src/llmserve/engine.py:29-72); it is an addition of this library.
 *
 * Who needs it.  lse_sample() wants a scratch buffer of rows * vocab floats from its caller.
 * Some callers cannot get one at the moment they sample: code that runs inside a region where
 * cudaMalloc is forbidden or would stall everything (a memory pool that has been frozen for the
 * serving phase, a plugin that is handed tensors but no allocator, a real-time loop that may not
 * take the driver's allocation lock, a process that has handed all device memory to a cache).
 * For them the library carries its own scratch: a fixed array in device memory that is part of
 * the loaded library image.  Every GPU on which this library is loaded holds those
 * LSE_SAMPLE_NOALLOC_MAX_FLOATS * 4 bytes (8 MiB) from load until the process exits.
 *
 * What it computes.  Exactly what lse_sample() computes (same kernel): for each of `rows` rows
 * of float32 `logits` (row r starts at logits + r * row_stride), temperature[r] <= 0 takes the
 * first largest logit; otherwise softmax(logits / temperature[r]), cut to the top_p[r] mass when
 * top_p[r] < 1, and the token at the inverse CDF (vocabulary order) of the counter-based uniform
 * number of (seed[r], counter[r]).  out[r] receives the token id.  All pointers are device
 * pointers supplied by the caller; the launch goes to `stream`.
 *
 * Limits and rules.
 *   - rows * vocab must not exceed LSE_SAMPLE_NOALLOC_MAX_FLOATS (for instance 13 rows of a
 *     151,936-token vocabulary, or 8 rows of 262,144).  A larger request is refused: the call
 *     returns LSE_SAMPLE_NOALLOC_TOO_LARGE, prints one line to stderr and launches nothing.
 *   - The call allocates nothing and frees nothing: no cudaMalloc, cudaFree or library routine
 *     that allocates.  The first call on a device looks up the address of the built-in scratch
 *     (cudaGetSymbolAddress, with that device current) and remembers it for later calls on that
 *     device.  Make that first call outside any stream capture.
 *   - All calls on a device share the one scratch array, and it keeps whatever the last call
 *     left in it.  Nothing in it has to start at zero: every value the kernel reads was written
 *     by the same launch first.  Two calls that overlap on the GPU (different streams, no
 *     ordering between them) race on the array and give wrong tokens; keep them ordered.
 *
 * Returns 0 on success, a positive cudaError_t value if CUDA reported an error, or one of the
 * negative codes below.
 */
#ifndef LSE_SAMPLING_NOALLOC_H
#define LSE_SAMPLING_NOALLOC_H

#include <cuda_runtime.h>

#define LSE_SAMPLE_NOALLOC_MAX_FLOATS (2 * 1024 * 1024)
#define LSE_SAMPLE_NOALLOC_BAD_ARGUMENT (-1)
#define LSE_SAMPLE_NOALLOC_TOO_LARGE (-2)

#ifdef __cplusplus
extern "C" {
#endif

int lse_sample_noalloc(const float* logits, long long row_stride, int rows, int vocab,
                       const float* temperature, const float* top_p, const long long* seed,
                       const long long* counter, int* out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif
