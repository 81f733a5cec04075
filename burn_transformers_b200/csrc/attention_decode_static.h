// bt_attention_decode_static: decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project (NoahIsCool/burn-transformers); it is an
// addition of this library.
//
// Who needs it.  Some programs that want to call this kernel are not free to obtain device memory: an
// operator loaded into a host runtime that owns the whole memory plan and hands a plug-in nothing but its
// input and output buffers; or a serving loop that has given all device memory to its own pool at start-up
// and forbids cudaMalloc afterwards, because a driver allocation stalls every stream of the device.  The
// ordinary entry point, bt_attention_decode, needs the caller to bring scratch memory for the partial
// results of its splits; such callers have nowhere to get it from.  This variant brings its own: a fixed
// array that is part of the library's image, BT_DECODE_STATIC_SCRATCH_FLOATS floats (4 MiB), which every
// GPU that loads the library holds until the process exits.
//
// What it does.  Exactly what bt_attention_decode does, with the same arguments minus `scratch`.  It calls
// no cudaMalloc, cudaFree or any allocating routine, its own or a library's.
//
// Limits and rules.
//  * n_seqs * n_heads * n_splits * (head_dim + 2) must not exceed BT_DECODE_STATIC_SCRATCH_FLOATS; a larger
//    request is refused with an error (bt_last_error() says by how much) and nothing is launched.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
//    current).  Make that first call before any stream capture begins on that device.
//  * n_seqs * n_heads must not exceed 16384 (the built-in ticket counters the splits' merge uses).
//  * All calls on a device share the one array, and the array keeps whatever the last call left in it.  The
//    kernels write every partial result they later read, so the partial results need no clearing.  The ticket
//    counters must be zero when a call starts: they are zero when the library is loaded, and the block that
//    merges a (sequence, head) sets its counter back to zero, so a completed call leaves them zero.  Two calls
//    that overlap on the GPU (different streams, no ordering between them) race on the array and give wrong
//    results: order them, or use bt_attention_decode with separate scratch buffers.
//  * The kernel's only wait (for its copies of cache pages to land) is bounded.  A block whose wait runs out
//    writes NaN as its result, still takes its ticket (so the counters return to zero) and sets a status word
//    that also lives inside the library.  bt_attention_decode_static_status copies that word to the host with
//    a blocking cudaMemcpy (0 = every wait was met) and clears it; it allocates nothing either.
#pragma once
#include <cuda_runtime.h>

#define BT_DECODE_STATIC_SCRATCH_FLOATS (1 << 20)

extern "C" int bt_attention_decode_static(const void* q, long long q_row_stride, const void* k_pool,
                                          const void* v_pool, const int* kv_table, int table_stride, int table_len,
                                          int page_size, void* out, const int* ctx_len, int n_seqs, int n_heads,
                                          int n_kv_heads, int head_dim, float scale, int window, int n_splits,
                                          int dtype, cudaStream_t stream);

// Reads (and clears) the status word of this device's bt_attention_decode_static calls into *status_out.
// Blocks until the device has finished the work queued before it.
extern "C" int bt_attention_decode_static_status(int* status_out);
