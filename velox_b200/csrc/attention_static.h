/* Decode attention over the paged cache that allocates nothing.
 *
 * This entry point has no counterpart in the reference project.  It exists for callers that
 * cannot allocate device memory while they run: a caller that hands all of the device's memory
 * to its own pool and must not let anything grow outside it, a caller on a thread where a
 * blocking allocation would stall other streams, or a C program that links the attention
 * library without torch and has no caching allocator at hand.  The ordinary launcher
 * (vx_attention) takes its scratch (the partial results of split key ranges and the counters
 * of the fused merge) from the caller, and the engine gets that from torch's allocator; this
 * one keeps the scratch in a fixed array inside the library, so a call makes no cudaMalloc,
 * no cudaFree and no call of an allocating library routine.
 *
 * What it computes is what vx_attention computes with kind 2 (the bfloat16 family with tiles of
 * 16 rows, for single decoded tokens and other short portions) and a fused merge: the same
 * kernel, the same work items (int32[8] each, at most 16 rows per item) and merge items, the
 * same results.  One library exists per head size; the limits below hold for each.
 *
 * Set-up.  The first call on a device finds the scratch array (cudaGetSymbolAddress), raises
 * the kernel's shared-memory limit and clears the counters.  That call synchronises with the
 * device, so make it once, early, before any stream capture begins; later calls only clear the
 * counters they use (a memset on `stream`) and launch the kernel.
 *
 * Sharing.  All calls of a process on one device share the one array.  Calls on one stream
 * follow each other and are safe.  Two calls that may overlap (different streams without an
 * event between them, or two threads) race on the scratch and give wrong results: order them.
 * The counters have to be zero when the kernel starts; every call clears those it uses before
 * its launch, so a call that was abandoned halfway leaves nothing behind for the next one.
 *
 * Limits.  A call whose split key ranges need more than
 * VX_ATTENTION_STATIC_MAX_PARTIAL_ROWS partial rows (over all KV heads), or more than
 * VX_ATTENTION_STATIC_MAX_COUNTERS counters (merge items x KV heads), is refused with
 * VX_ATTENTION_STATIC_TOO_LARGE and a message; nothing is launched.  The array takes
 * MAX_PARTIAL_ROWS * (head size + 1) * 4 + MAX_COUNTERS * 4 bytes of device memory per loaded
 * library (4.2 MB at head size 128).  A decode step of 64 sequences on 2 KV heads whose key
 * ranges are cut into 4 splits of 7 query heads each needs 64 * 4 * 2 * 7 = 3,584 rows.
 */
#ifndef VELOX_B200_ATTENTION_STATIC_H_
#define VELOX_B200_ATTENTION_STATIC_H_

#include <cuda_runtime_api.h>

#define VX_ATTENTION_STATIC_MAX_PARTIAL_ROWS 8192
#define VX_ATTENTION_STATIC_MAX_COUNTERS 4096

/* Return values besides 0 (launched) and positive cudaError_t codes. */
#define VX_ATTENTION_STATIC_TOO_LARGE (-2)
#define VX_ATTENTION_STATIC_BAD_ARGUMENT (-3)

#ifdef __cplusplus
extern "C" {
#endif

/* q [T, q_stride] and out [T, out_stride] bfloat16; k_cache, v_cache [num_pages, page_size,
 * num_kv_heads, head size] bfloat16; block_tables [sequences, table_stride]; q_start, q_len,
 * kv_len one int per sequence; items [num_items, 8]; merge_items [num_merges, 8] (may be null
 * when num_merges is 0); partial_rows: the rows the items' partial_base fields span (0 if no
 * item is split).  The items stay on the device and are not read by this function, so
 * partial_rows is taken on the caller's word for the size check; should an item all the same
 * name a row beyond VX_ATTENTION_STATIC_MAX_PARTIAL_ROWS, the kernel writes nothing for it and
 * sets bit 32 of *status.  The items must come from a plan made for the same num_kv_heads and
 * group (row = partial_base + kv_head * row_count + r).  status: one int on the device that
 * collects the kernels' error bits.
 * error (may be null) receives a zero-terminated message of at most error_capacity bytes
 * when the return value is not 0. */
__attribute__((visibility("default"))) int vx_attention_decode_static(
    const void* q, void* out, const void* k_cache, const void* v_cache, const int* block_tables,
    const int* q_start, const int* q_len, const int* kv_len, const int* items, int num_items,
    const int* merge_items, int num_merges, int partial_rows, int* status, int q_stride,
    int out_stride, int table_stride, int num_kv_heads, int group, int page_size,
    long long num_pages, int window, float softmax_scale, cudaStream_t stream, char* error,
    int error_capacity);

#ifdef __cplusplus
}
#endif

#endif /* VELOX_B200_ATTENTION_STATIC_H_ */
