/* Decode attention for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference project; it exists for hosts of this
 * library that cannot call cudaMalloc at the moment they need attention:
 *   - a serving process that handed every free byte of the GPU to its own pools at start-up
 *     (this engine's cache does exactly that), so a later cudaMalloc would simply fail;
 *   - a latency-critical loop in which the implicit device synchronisation of an allocation
 *     (or of the matching cudaFree) is not acceptable.
 * The split-KV decode kernel needs scratch memory for the partial results of its key splits and
 * one ticket per (row, head). The ordinary entry point (ayk_attention_decode) takes that
 * scratch from the caller; this one keeps it in a fixed array inside the library instead:
 *
 *   AYK_NOALLOC_PARTIAL_FLOATS = 1,048,576 floats (4 MiB)  >= rows * heads * splits * (head_dim + 2)
 *   AYK_NOALLOC_TICKETS        =    16,384 ints  (64 KiB)  >= rows * heads
 *
 * Every GPU that loads the library holds this array (about 4.1 MiB) until the process exits.
 * A call whose sizes exceed either limit is refused with AYK_TOO_LARGE (-3) and launches
 * nothing; ayk_attention_decode_noalloc_limits() reports the two limits.
 *
 * What the caller must know:
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress,
 *     with that device current) and remembers it. Make that first call outside any stream
 *     capture, and before the host gives the device's free memory away: the driver may load
 *     the library's device image, the array included, only at that first use, and that load
 *     needs the 4.1 MiB to be free. If it fails the call returns the CUDA error and a later
 *     call tries again.
 *   - All calls share the one array. It keeps whatever the last call left; the entry point
 *     zeroes the tickets it is about to use on the caller's stream before every launch, and
 *     every partial result is written before it is read, so stale contents never matter.
 *     Two calls that overlap on the GPU (different streams, no dependency) race on the array:
 *     serialise them.
 *   - Nothing here calls cudaMalloc, cudaFree or any allocating library routine; inputs and
 *     outputs are the caller's.
 *
 * Arguments are those of ayk_attention_decode without the scratch and fused-store arguments:
 * q/out [rows, heads * head_dim] (row strides ld_q/ld_out, in elements), paged keys and values
 * [page][kv_head][slot][head_dim], block_table [*, table_stride] int32 (0 = no page),
 * request_of_row/positions [rows] int32, type 0 = float32, 1 = bfloat16, stream a cudaStream_t.
 * Returns 0, a negative refusal code (see common.cuh) or a positive cudaError_t.
 */
#pragma once

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

int ayk_attention_decode_noalloc(const void* q, int ld_q, const void* k_pages,
                                 const void* v_pages, const int* block_table, int table_stride,
                                 const int* request_of_row, const int* positions, void* out,
                                 int ld_out, int num_rows, int num_heads, int num_kv_heads,
                                 int head_dim, int page_size, float scale, int window,
                                 int splits, int type, void* stream);

void ayk_attention_decode_noalloc_limits(size_t* partial_floats, size_t* tickets);

#ifdef __cplusplus
}
#endif
