// Split-KV decode attention that allocates nothing.
//
// This entry point has no counterpart in the reference (ermolushka/rvllm); it exists
// for callers of this library that are not able to allocate device memory themselves:
// a plug-in that runs inside a host program which handed every byte of the device to
// its own pool at start-up, a control loop that must not take the device-wide stall a
// cudaMalloc or cudaFree can cause, or a C program that links this library without
// torch and therefore has no caching allocator to ask for the scratch buffer that
// `rv_paged_attention_decode` wants from its caller.
//
// It computes exactly what `rv_paged_attention_decode` computes (same kernels, same
// order of sums), but the partial results of the key splits live in a fixed array that
// is part of the library image instead of a caller-provided buffer.
//
//   * The array is RV_DECODE_STATIC_SCRATCH_BYTES (4 MiB) large.  Every GPU on which
//     the library's kernels are loaded holds these 4 MiB until the process exits.
//   * A call whose partial results need more than that is refused with an error
//     message; nothing is launched.  The need is
//         n_reqs * num_heads * ceil(max_ctx_len / 256) * (head_dim * 4 + 8) bytes,
//     so for example 8 requests x 32 heads x 4,096 tokens x head size 64 need 1.03 MiB.
//   * The first call on a device looks up the array's device address (with that device
//     current) and remembers it; make that first call outside any stream capture.
//     Later calls on the same device only launch kernels.
//   * The function calls no cudaMalloc, cudaFree or any library routine that allocates.
//   * All calls share the one array, and it keeps what the last call left in it.  Nothing
//     in it has to start at zero: each call writes every partial result before the merge
//     kernel reads it.  Two calls that overlap on the GPU (different streams, no
//     dependency between them) race on the array; run them on one stream or order them
//     with events.
//
// Inputs and outputs are the caller's, as for `rv_paged_attention_decode`:
//   q            [n_reqs, q_stride] rows whose first num_heads * head_dim elements are the
//                queries (one token per request), dtype code 0 = float32, 1 = bfloat16
//   k_cache,     [pages, page_size, num_kv_heads, head_dim], same dtype
//   v_cache
//   block_table  int32 [n_reqs, max_blocks], page ids of each request
//   ctx_lens     int32 [n_reqs], tokens in the cache including the current one; 0 skips.
//                Every entry must be <= max_ctx_len: the launch covers max_ctx_len keys, and
//                a request that claims more gets NaN in its output rows instead of a result
//                that silently leaves keys out.
//   out          [n_reqs, num_heads * head_dim], same dtype
//   window       0 for none, else only the last `window` keys are visible
// Returns 0, or non-zero with the reason in rv_last_error().
#pragma once

#define RV_DECODE_STATIC_SCRATCH_BYTES (4 << 20)

#ifdef __cplusplus
extern "C" {
#endif

int rv_paged_attention_decode_static(const void* q, int dtype, int q_stride, const void* k_cache,
                                     const void* v_cache, const int* block_table, int max_blocks,
                                     const int* ctx_lens, void* out, int n_reqs, int max_ctx_len,
                                     int num_heads, int num_kv_heads, int head_dim, int page_size,
                                     float scale, int window, void* stream);

// Bytes of the fixed array a call with these sizes would use.
long long rv_paged_attention_decode_static_need(int n_reqs, int num_heads, int head_dim,
                                                int max_ctx_len);

#ifdef __cplusplus
}
#endif
