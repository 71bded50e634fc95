// Split paged decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference: the reference's
// launcher allocates three scratch buffers on every call
// (crates/vllm-cuda/src/kernels/paged_attn_op.rs:98-140).
//
// Who needs it: code that runs where cudaMalloc is off limits -- a host
// program that has handed all device memory to its own pool and must not
// fragment it, a plugin called from inside another runtime's stream callback
// or real-time loop where an allocation (which may synchronise the device)
// is forbidden, or a C caller that has no tensor library to allocate with.
// Such a caller passes only inputs and outputs; the partial results of the
// split kernel live in a fixed array inside this library.
//
// The scratch is a file-scope __device__ array of RG_STATIC_SCRATCH_BYTES
// (4 MiB).  Every GPU that loads the library holds those 4 MiB until the
// process exits.  With S = n_tokens * num_heads * num_splits, a call needs
//     4 * (round64(S * head_dim) + round64(S * 2)
//          + n_tokens * num_kv_heads * ceil(num_heads / num_kv_heads / 8)) bytes,
// round64 rounding up to a multiple of 64 (the partial outputs, the partial
// maxima and sums, and one counter per token, key/value head and tile of 8
// query heads).  A call that needs more is refused with
// RG_ERR_SCRATCH_TOO_LARGE and a message, and nothing is launched.
//
// The first call on a device looks up the array's device address
// (cudaGetSymbolAddress; the array's name in host code is only a stand-in,
// not an address a kernel could use).  Make that first call before any stream
// capture begins.  Later calls do no set-up.
//
// All calls share the one array and it keeps the last call's contents.  The
// kernels write every partial result they later read; the counters that tell
// the last block of a token to reduce must be zero on entry, and since their
// place in the array depends on the sizes and may hold an earlier call's partial
// results, every call clears its own counters first (cudaMemsetAsync on the
// caller's stream, no allocation).  Two calls whose kernels overlap on the GPU
// (different streams, no ordering between them) race on the array.  Order them.
//
// It calls no cudaMalloc, cudaFree or allocating library routine.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define RG_STATIC_SCRATCH_BYTES (4u << 20)
#define RG_ERR_SCRATCH_TOO_LARGE 10002

// Arguments as rg_decode_attention's, without the two scratch pointers:
//   q            bfloat16, rows q_stride elements apart, head h at offset h * head_dim
//   out          bfloat16 [tokens, num_heads * head_dim]; rows listed in `rows` are written
//   kv_cache     bfloat16 [pages, 2, num_kv_heads, page_size, head_dim]
//   block_table  int32 [requests, max_blocks]
//   rows         int32 [n_tokens] token rows to compute, or NULL for rows 0 .. n_tokens-1
//   req_of_token int32 [tokens] request index of every token row
//   positions    int32 [tokens] absolute position of every token row
//   error_text   NULL, or a buffer of error_cap bytes that receives a message when the result is not 0
// Returns 0, RG_ERR_SCRATCH_TOO_LARGE, 10001 (sizes the kernels refuse) or a cudaError_t.
int rg_decode_attention_static_scratch(
    const void* q, int q_stride, void* out, const void* kv_cache, const int* block_table, int max_blocks,
    const int* rows, int n_tokens, const int* req_of_token, const int* positions,
    int num_heads, int num_kv_heads, int head_dim, int page_size, int window, float scale, int num_splits,
    void* stream, char* error_text, int error_cap);

#ifdef __cplusplus
}
#endif
