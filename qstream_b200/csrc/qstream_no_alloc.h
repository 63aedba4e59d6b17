/* qstream_no_alloc.h - decode attention for callers that must not allocate.
 *
 * This entry point has no counterpart in QStream (the reference engine is CPU-only and
 * owns one arena); it exists for this library's GPU callers.
 *
 * Who needs it: code that runs where device memory cannot be obtained or released - a
 * caller that holds a fixed memory plan and has handed every byte to someone else, a
 * plug-in loaded into a process whose allocator it may not touch, code inside a region
 * where cudaMalloc is forbidden or would synchronise the device (a latency-critical
 * loop, a stream that is being captured).  The ordinary entry point
 * `qs_attention_decode` asks its caller for a scratch buffer for the partial results
 * of the key splits; such callers have nowhere to get one from.
 *
 * `qs_attention_decode_static` is the same computation with that scratch taken from a
 * fixed array inside the library.  The caller passes inputs and outputs only.
 *
 *  - Limit: the scratch holds QS_DECODE_STATIC_SCRATCH_FLOATS floats (4 MiB).  A call needs
 *    T_tokens * n_heads * ceil(max_context / 256) * (head_dim + 2) floats; a larger call is
 *    refused with QS_ERR_INVALID_INPUT (11) and a message in qs_last_error(), nothing runs.
 *  - Cost: every GPU that loads the library holds these 4 MiB until the process exits.
 *  - First call on a device: the library looks up the array's device address once per
 *    device (cudaGetSymbolAddress, with that device current) and remembers it.  Make the
 *    first call on each device outside any stream capture.
 *  - The function calls no cudaMalloc, cudaFree or other allocating routine.
 *  - Sharing: all calls on a device use the same array, which keeps what the last call
 *    left in it.  Nothing in it has to start at zero (every element that is read has been
 *    written earlier in the same call), so nothing is cleared.  Two calls whose kernels may
 *    overlap on the GPU (different streams, no ordering between them) race on the array and
 *    give wrong results; calls on one stream, or ordered by events, are safe.
 *
 *  - Bounds the caller keeps: every `tok_pos[t]` lies in [0, max_context rounded up to 256) -
 *    a position outside sets the status word to 1 and gives that row zeros, nothing is read
 *    for it; every `tok_slot[t]` is negative (a padding row: zeros) or a row of `page_table`.
 *
 * Arguments are those of `qs_attention_decode` without `scratch`.
 */
#ifndef QSTREAM_NO_ALLOC_H
#define QSTREAM_NO_ALLOC_H

#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QS_DECODE_STATIC_SCRATCH_FLOATS (1 << 20)

int qs_attention_decode_static(void* out, long long ldo, const void* q, long long ldq,
                               const void* k_cache, const void* v_cache,
                               const int32_t* page_table, int max_pages, int page_tokens,
                               const int32_t* tok_slot, const int32_t* tok_pos, int T_tokens,
                               int n_heads, int n_kv_heads, int dh, float scale, int window,
                               int max_context, int32_t* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* QSTREAM_NO_ALLOC_H */
