// ps_paged_attention_decode_noalloc: split-key paged attention that allocates nothing.
//
// This entry point has no counterpart in the reference (jainalphin/pagedserve); it is an addition
// of this library.
//
// Who it is for. ps_paged_attention_decode needs scratch memory whenever the keys of a token are
// split over several CTAs, and leaves it to the caller to provide it. Some callers cannot: a host
// program that gave the whole device to its own pool at start-up and must not call cudaMalloc later
// (the call may fail, and it stalls the device while it runs); a caller outside Python that has no
// allocator of ours to ask; a latency-critical loop that is not allowed to touch the allocator at
// all. For them this variant keeps the scratch in a fixed array that is part of the library image.
//
// What it costs. The array is PS_NOALLOC_SCRATCH_BYTES (4,243,712 bytes) of device memory on every
// GPU that loads the library, held until the process exits, whether or not the entry point is used.
//
// Limits (beyond them the call is refused with PS_ERR_SCRATCH_LIMIT and a message, nothing runs):
//   T * n_heads            <= PS_NOALLOC_MAX_ROWS      (4096)   one counter per (token, head)
//   T * n_heads * n_splits <= PS_NOALLOC_MAX_PARTIALS  (4096)   one partial state per split
//   head_dim               <= 256
//
// Rules for the caller.
//   * Inputs and outputs are still the caller's memory; only the scratch is ours.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress) with
//     that device current. Make that first call before any stream capture begins.
//   * Every call on a device shares the one array. The counters are cleared at the start of each
//     call; the partial states keep the previous call's contents until they are overwritten. Two
//     calls that overlap on the GPU (different streams, no ordering between them) race on it: order
//     them yourself.
//   * No cudaMalloc, cudaFree or allocating library routine is called, by this entry point or by
//     anything it uses.
//   * The split rule is the caller's: a split is split_tiles * 32 keys (a whole number of the
//     kernel's chunks: 128 keys up to head size 64, 64 up to 128, 32 above, never fewer than a
//     page), and n_splits must reach every token's newest key: n_splits >= floor(longest position
//     / (split_tiles * 32)) + 1. A token that the grid does not reach gets no output.
//   * The kernel reports what it cannot report through the return code (the grid did not reach a
//     token: 3; a bounded wait inside the kernel ran out: 2) in one status word at the end of the
//     fixed array. ps_paged_attention_decode_noalloc_status copies it to the host (and clears it
//     if asked) on the given stream and waits for that stream; 0 means every call since the last
//     clear was fine. It allocates nothing either.
//
// Arguments are those of ps_paged_attention_decode without the three scratch pointers, plus an
// optional buffer that receives a readable message when the call is refused.
#pragma once

#define PS_NOALLOC_MAX_ROWS 4096
#define PS_NOALLOC_MAX_PARTIALS 4096
#define PS_NOALLOC_MAX_HEAD_DIM 256
// counters | (max, sum) pairs | partial accumulators | status word (padded to 256 bytes)
#define PS_NOALLOC_STATUS_OFFSET \
    (PS_NOALLOC_MAX_ROWS * 4 + PS_NOALLOC_MAX_PARTIALS * 2 * 4 + PS_NOALLOC_MAX_PARTIALS * PS_NOALLOC_MAX_HEAD_DIM * 4)
#define PS_NOALLOC_SCRATCH_BYTES (PS_NOALLOC_STATUS_OFFSET + 256)
#define PS_ERR_SCRATCH_LIMIT 4
#define PS_ERR_SETUP 5

#ifdef __cplusplus
extern "C" {
#endif

int ps_paged_attention_decode_noalloc(const void* q, int q_stride, void* out, int out_stride,
                                      const void* k_pool, const void* v_pool, long long page_stride,
                                      const int* token_item, const int* positions, const int* block_table,
                                      int bt_stride, int T, int n_heads, int n_kv_heads, int head_dim,
                                      int page_size, int window, float scale, int split_tiles, int n_splits,
                                      void* stream, char* message, int message_capacity);

// *value = the status word of the fixed array on the current device; clear != 0 also zeroes it.
int ps_paged_attention_decode_noalloc_status(int* value, int clear, void* stream);

#ifdef __cplusplus
}
#endif
