// ie_attention_decode_static -- paged decode attention for callers that cannot allocate.
//
// This entry point has no counterpart in the reference: it is an addition of this library.
//
// Who it is for.  Some hosts of this library are not allowed to call cudaMalloc (or any
// routine that allocates device memory on their behalf) at the point where they run attention:
// a plugin inside a runtime that owns all device memory and hands out none, code running
// while the memory pool is frozen, or a latency-critical loop whose owner forbids allocator
// calls.  The regular entry point, ie_attention_decode, needs scratch memory for the partial
// results of its context splits and expects the caller to bring it.  This variant brings its
// own: a fixed array compiled into the library's device image.
//
// What it does.  Exactly what ie_attention_decode does (same kernels, same results) for
// requests with at most 16 rows (tokens x query heads per key/value head).  Inputs and outputs
// are still the caller's.  It calls no cudaMalloc, cudaFree or allocating library routine.
//
// Limits and rules.
//   * The scratch array holds IE_STATIC_DECODE_SCRATCH_FLOATS floats (4 MiB).  The attention
//     library is built once per head size (libie_b200_attn_hd<N>), and each of them carries an
//     array of its own: a process holds 4 MiB per loaded head-size library on every GPU it
//     uses, not 4 MiB in all.  A call needs
//     num_seqs * nkv * num_splits * 16 * (head_dim + 2) floats when num_splits > 1 and none
//     when num_splits == 1.  A call that needs more is refused with
//     IE_STATIC_SCRATCH_TOO_SMALL and a message that says how much was asked for; nothing is
//     launched.  Every GPU that loads the library holds the array until the process exits.
//   * The first call with num_splits > 1 on a device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current; the address is kept per device).
//     Make that first call outside any stream capture.
//   * A second small array (IE_STATIC_DECODE_MAX_TICKETS ints) holds one ticket counter per
//     request and key/value head, by which the last block to finish knows it has to merge the
//     splits.  Counters must be zero when the kernel starts: every call clears the ones it
//     uses (cudaMemsetAsync on the caller's stream) before the launch.  num_seqs * nkv beyond
//     that count is refused like too large a scratch need.
//   * All calls share the arrays, and they keep what the last call left.  The partial results
//     need no clearing: a call writes every partial it later reads.  Because they are shared,
//     two calls whose kernels can overlap on the GPU (different streams, no dependency) race
//     on it; run such calls on one stream or order them with events.
//   * What must be complete before the call.  The kernel is launched so that it may start
//     while the kernel before it on the stream is still finishing (programmatic stream
//     serialization), and it reads `cu_q`, `ctx_lens`, `tables` and the cached keys and values
//     of earlier positions before it waits for that kernel; only `q` and the newest position's
//     keys and values are read after the wait.  So if the kernel directly before this call on
//     the stream writes lengths, tables or older cache entries, either that kernel must not
//     signal its dependents early (kernels that never call griddepcontrol.launch_dependents,
//     and copies, do not), or switch the early start off for this library with ie_set_pdl(0).
//   * Kernel set-up (shared-memory limit, SM count) is kept per device, like the array's
//     address: the entry point may be used on several GPUs of one process.
//   * `msg`, if not null, receives a zero-terminated explanation when the return value is
//     not 0 (at most msg_len bytes).
#pragma once

#define IE_STATIC_DECODE_SCRATCH_FLOATS (1 << 20)
#define IE_STATIC_DECODE_MAX_TICKETS 8192
#define IE_STATIC_SCRATCH_TOO_SMALL (-1001)

#ifdef __cplusplus
extern "C" {
#endif

// Floats the built-in scratch array holds.
long long ie_attention_decode_static_capacity_floats(void);

// q [tokens, nh * head_dim], out likewise (bfloat16); k_cache, v_cache
// [pages, nkv, page_size, head_dim] (bfloat16); tables [num_seqs, table_width] int32 (page of
// every 'page_size' positions); cu_q [num_seqs + 1] first token of each request; ctx_lens
// [num_seqs] tokens cached after this step; err: 4 ints of device memory for index-check
// reports, or null; stream: a cudaStream_t.  Returns 0, a cudaError_t, or
// IE_STATIC_SCRATCH_TOO_SMALL.
int ie_attention_decode_static(const void* q, const void* k_cache, const void* v_cache,
                               const int* tables, int table_width, const int* cu_q,
                               const int* ctx_lens, void* out, int num_seqs, int nh, int nkv,
                               int page_size, int total_pages, float scale, int window,
                               int num_splits, int* err, void* stream, char* msg, int msg_len);

#ifdef __cplusplus
}
#endif
