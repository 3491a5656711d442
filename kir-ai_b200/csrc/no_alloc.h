/* Decode attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in michaelasper/kir-ai; it is an addition of this
 * library.
 *
 * Who needs it.  The split-KV decode kernel passes partial results between two launches
 * through scratch memory, and kirai_attention_decode_bf16 asks its caller for that buffer.
 * A caller written against torch gets it from torch's caching allocator.  A caller without
 * such an allocator may have no way to provide one in the middle of a step: a serving
 * process that handed every free byte of the device to its cache pool at start-up gets an
 * out-of-memory error from a later cudaMalloc, and cudaMalloc/cudaFree may also stall the
 * whole device while they run, which a step loop with latency bounds cannot accept.  Some
 * hosts forbid allocation after start-up outright.
 *
 * What it does instead.  The scratch lives in a file-scope array of the library,
 * KIRAI_STATIC_SCRATCH_FLOATS floats (4 MiB), aligned to 256 bytes.  Every GPU that loads
 * the library holds these 4 MiB until the process exits.  The caller still passes inputs
 * and outputs.  The function calls no cudaMalloc, cudaFree or any other allocating routine.
 *
 * Limits and rules.
 *  - requests * q_heads * num_splits * (head_dim + 2) must not exceed
 *    KIRAI_STATIC_SCRATCH_FLOATS; otherwise nothing is launched and
 *    KIRAI_ERR_STATIC_SCRATCH_TOO_SMALL is returned.  (With num_splits == 1 no scratch is used.)
 *  - The first call on a device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current) and remembers it; make that first call
 *    before any stream capture begins on that device.
 *  - All calls share the one array, and it keeps what the last call left.  Nothing has to be
 *    cleared: a call writes every word that its second launch reads.  Two calls that may run
 *    on the GPU at the same time (different streams, no ordering between them) race on the
 *    array and must not be issued; calls in one stream are ordered and safe.
 *  - Other return values and all arguments are those of kirai_attention_decode_bf16.
 */
#ifndef KIRAI_NO_ALLOC_H
#define KIRAI_NO_ALLOC_H

#include <cuda_runtime.h>

#define KIRAI_STATIC_SCRATCH_FLOATS (1u << 20)
#define KIRAI_ERR_STATIC_SCRATCH_TOO_SMALL (-5)
#define KIRAI_ERR_STATIC_SCRATCH_SETUP (-6)

#ifdef __cplusplus
extern "C" {
#endif

int kirai_attention_decode_bf16_static_scratch(const void* q, const void* cache, void* out, const int* block_table,
                                               const int* context_len, int requests, int q_heads, int kv_heads,
                                               int head_dim, long q_row_stride, int page_size, int table_width,
                                               int num_pages, int window, float scale, int num_splits,
                                               int* error_flag, cudaStream_t stream);

/* KIRAI_STATIC_SCRATCH_FLOATS, for callers that load the library without this header. */
unsigned kirai_static_scratch_capacity_floats(void);

#ifdef __cplusplus
}
#endif
#endif
