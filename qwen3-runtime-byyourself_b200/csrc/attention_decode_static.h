// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (RicardoMin/Qwen3-Runtime-ByYourself);
// it is an addition of this library.
//
// Who needs it: code that runs where cudaMalloc is not an option - inside a region whose
// memory was handed out up front (a serving process with a fixed budget per model, a plugin
// that lives in somebody else's allocator), in a callback or a latency-critical loop where an
// allocation could synchronise the device, or in a host program that simply has no allocator
// to pass scratch from.  The regular entry point, q3_attention_decode_bf16, asks its caller
// for a float32 scratch buffer in which the partial results of the key splits meet; this
// variant keeps that buffer inside the library, in a fixed device array.
//
// Limit: the array holds Q3_DECODE_STATIC_MAX_FLOATS float32 values (8 MiB).  A call needs
//     n_tokens * nq * n_splits * (head_dim + 2)
// of them and is refused with Q3_ERR_STATIC_SCRATCH (and one line on stderr) if that is more.
// Every GPU on which the library is used holds the 8 MiB until the process exits.
//
// Rules of use:
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress)
//     and sets the kernel's shared-memory attribute.  Make that first call outside any
//     stream capture, with the device current that the call is meant for.  `stream` has to be
//     a stream of the current device: the array's address is looked up for that device, and
//     nothing here can tell which device a stream belongs to.  Host threads may make their
//     first calls at the same time (the set-up is guarded); the rule on overlapping calls
//     below holds for threads as it does for streams.
//   * All calls share the one array.  Nothing in it has to be zero: every slot a call reads
//     it has written before, so the previous call's contents do no harm.  Two calls that
//     overlap on the GPU (different streams, or graphs replayed concurrently) race on it;
//     run them in stream order.
//   * Nothing is allocated or freed: no cudaMalloc, no cudaFree, no library workspace.
//   * The library is compiled for one head size (-DQ3_HEAD_DIM=...), like the regular one.
#pragma once
#include <stdint.h>

#define Q3_DECODE_STATIC_MAX_FLOATS (2 * 1024 * 1024)
#define Q3_ERR_STATIC_SCRATCH 10004

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as q3_attention_decode_bf16, without the scratch pointer:
//   q [n_tokens, nq, head_dim] bf16, k_pages / v_pages [pages, nkv, 64, head_dim] bf16,
//   out [n_tokens, nq, head_dim] bf16, token_seq / token_pos [n_tokens] int32,
//   page_table [sequences, pages_per_seq] int32, all device pointers; `stream` a cudaStream_t.
// Returns 0, a cudaError_t, Q3_ERR_BAD_SIZE (10001) / Q3_ERR_TOO_LARGE (10002) for sizes the kernel
// does not take, or Q3_ERR_STATIC_SCRATCH when the call needs more than the built-in scratch.
int q3_attention_decode_bf16_static(const void* q, const void* k_pages, const void* v_pages, void* out,
                                    const int* token_seq, const int* token_pos, const int* page_table,
                                    int pages_per_seq, int64_t n_tokens, int nq, int nkv, float scale, int window,
                                    int n_splits, void* stream);

#ifdef __cplusplus
}
#endif
