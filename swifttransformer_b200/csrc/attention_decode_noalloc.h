// st_attention_decode_noalloc: split paged decode attention for callers that
// cannot allocate device memory.
//
// This entry point has no counterpart in LLMServe/SwiftTransformer; it exists
// for hosts that embed this library but must not let it call cudaMalloc.  Such
// callers exist for ordinary reasons: a serving process that hands its whole
// device-memory budget to its own pool at start-up and forbids later
// allocations so that it can never fail with out-of-memory mid-request; code
// that runs between the begin and end of a stream capture, where an allocation
// is an error; a real-time loop that may not take the device-wide
// synchronisation a cudaMalloc or cudaFree implies; and plug-in interfaces
// (a C host calling through this symbol with ctypes, dlopen or an FFI) that
// have no allocator to lend.  The regular entry point, st_attention_decode,
// needs a scratch buffer for the partial results of the key-range splits and a
// zeroed counter array from its caller; here both live inside the library, in a
// file-scope `static __device__` array of fixed size.
//
// What the caller still passes: the queries, the page pool, the block table
// and index arrays, and the output buffer - exactly the arguments of
// st_attention_decode without `partial` and `counters`.
//
// Limits and rules
//   * The built-in scratch holds ST_NOALLOC_SCRATCH_FLOATS floats (4 MiB) for
//     partial results and ST_NOALLOC_MAX_PAIRS (token, head) pairs.  A call
//     that needs more - n_items * nh * n_splits * (head_dim + 2) floats, or
//     n_items * nh pairs - is refused with ST_ERR_TOO_LARGE and a message in
//     `err`; nothing is launched.
//   * Every GPU that loads the library carries the array until the process
//     exits (about 4.1 MiB per device).
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and remembers it; make
//     that first call outside any stream capture.  Later calls only enqueue a
//     memset of the counters and the kernels on `stream`.
//   * All calls on a device share the one array.  Each call clears the
//     counters it uses and overwrites the partial results it needs, so calls
//     that run one after the other (same stream, or ordered by events) are
//     independent; two calls that overlap on the GPU race on the array and
//     give wrong results.
//   * The first call on a device also fills that device's entry of a small
//     table of addresses, without a lock: let one host thread make the first
//     call on a device before other threads call for the same device.
//   * It calls no cudaMalloc, cudaFree or allocating library routine.
//
// Returns 0, a positive cudaError_t, or a negative code: ST_ERR_TOO_LARGE (-3)
// when the call does not fit the built-in scratch, ST_ERR_BAD_ARG (-4) for
// sizes that make no sense, ST_ERR_BAD_SIZE (-2) for a head size the kernel
// does not take.  `err` may be null; otherwise up to err_len - 1 characters of
// explanation are written.
#pragma once

#ifndef ST_ERR_BAD_SIZE
#define ST_ERR_BAD_SIZE (-2)
#endif
#ifndef ST_ERR_TOO_LARGE
#define ST_ERR_TOO_LARGE (-3)
#endif
#ifndef ST_ERR_BAD_ARG
#define ST_ERR_BAD_ARG (-4)
#endif

#define ST_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define ST_NOALLOC_MAX_PAIRS 16384

#ifdef __cplusplus
extern "C" {
#endif

int st_attention_decode_noalloc(const void* q, const void* pool, void* out, const int* items, int n_items,
                                const int* positions, const int* seq_of_token, const int* slots,
                                const int* block_table, int max_pages, int n_layers, int layer, int nh, int nkv,
                                int d, int page_size, float scale, int window, int n_splits, void* stream,
                                char* err, int err_len);

#ifdef __cplusplus
}
#endif
