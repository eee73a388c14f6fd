// hos_attn_decode_noalloc: decoding attention over the paged cache for callers that must not
// allocate device memory.  (It has no counterpart in the reference, which has no GPU path for
// this model at all; it exists for embedders of this library.)
//
// Who needs it.  `hos_attn_decode` splits a long sequence's keys over several CTAs and needs a
// workspace for their partial results, which its Python face takes from torch's allocator.
// Some callers cannot do that: a serving loop that has handed all device memory to its own
// pool (an allocation may then fail, and cudaMalloc / cudaFree synchronise the whole device,
// which such a loop cannot afford in the middle of a step), or a plugin that runs inside
// another framework's memory allowance and was given input and output buffers and nothing else.
// For them the workspace lives inside the library: a file-scope `static __device__` array of
// HOS_NOALLOC_SCRATCH_BYTES (8 MiB) plus 16 KiB of counters, which every GPU that loads the
// library holds until the process ends.
//
// Contract.
//  * Same arguments and result as `hos_attn_decode` without the workspace and ticket
//    pointers; the caller still owns q, out, the cache pages and the index arrays.
//  * It calls no cudaMalloc, cudaFree or allocating library routine.  The first call on a
//    device looks up the device address of the scratch array (cudaGetSymbolAddress, with that
//    device current) and raises the kernel's shared-memory limit; make that first call before
//    any stream capture begins.
//  * Sizes whose partial results would not fit the scratch array (n_tokens * n_heads *
//    n_splits * (head_dim + 2) floats > 8 MiB, or more (token, kv head) pairs than 4096
//    counters) are refused with a message; nothing is launched.
//  * All calls share the one array.  It keeps what the last call left; the counters, which must
//    start at zero, are cleared on the caller's stream before every launch.  Two calls whose
//    kernels overlap on the GPU (different streams without an order between them) race on it:
//    keep calls on one stream or order them yourself.
//  * Where the shares of a step run as clusters that merge through shared memory (up to 16 shares, all
//    clusters on the GPU at once) the scratch array is not touched at all.
#pragma once
#include <cuda_runtime.h>

#define HOS_NOALLOC_SCRATCH_BYTES (8u << 20)
#define HOS_NOALLOC_TICKETS 4096

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0, or a negative code with the reason in hos_last_error().
int hos_attn_decode_noalloc(const void* q, int q_stride, void* out, int out_stride,
                            const int* token_pos, const int* token_seq, const int* seq_slot,
                            void* k_pages, void* v_pages, const int* page_table, int table_stride,
                            int ring_pages, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                            float scale, float cap, int window, int n_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
