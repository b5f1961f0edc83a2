// The allocation-free variant of split-KV decode attention: see
// attention_decode_static.h for who needs it and for its limits.
#include "attention_decode_static.h"

#include <mutex>

#include "common.cuh"

// The launcher that takes its scratch from the caller (attention_simt.cu).
extern "C" long long rv_paged_attention_decode_scratch_bytes(int n_reqs, int num_heads, int hd,
                                                             int max_ctx_len);
extern "C" int rv_paged_attention_decode(const void* q, int dtype, int q_stride,
                                         const void* k_cache, const void* v_cache,
                                         const int* block_table, int max_blocks,
                                         const int* ctx_lens, void* out, void* scratch,
                                         long long scratch_bytes, int n_reqs, int max_ctx_len,
                                         int num_heads, int num_kv_heads, int hd, int page_size,
                                         float scale, int window, void* stream);

// Partial results of the key splits.  In host code this name is only a stand-in for the
// symbol, not a device address: the address each device gave the array is looked up
// below and that pointer is what the kernels get.
static __device__ __align__(256) unsigned char g_decode_scratch[RV_DECODE_STATIC_SCRATCH_BYTES];

#define RV_MAX_DEVICES 64
static void* g_scratch_address[RV_MAX_DEVICES];   // per device, null until looked up
static std::mutex g_setup_lock;

// The array's address on the current device; looked up once per device.
static int scratch_address(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess)
        RV_FAIL("paged_attention_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= RV_MAX_DEVICES)
        RV_FAIL("paged_attention_decode_static: device %d is beyond the %d this library tracks",
                dev, RV_MAX_DEVICES);
    std::lock_guard<std::mutex> guard(g_setup_lock);
    if (!g_scratch_address[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_decode_scratch);
        if (e != cudaSuccess || !p)
            RV_FAIL("paged_attention_decode_static: cudaGetSymbolAddress: %s",
                    cudaGetErrorString(e));
        g_scratch_address[dev] = p;
    }
    *out = g_scratch_address[dev];
    return 0;
}

extern "C" long long rv_paged_attention_decode_static_need(int n_reqs, int num_heads,
                                                           int head_dim, int max_ctx_len) {
    return rv_paged_attention_decode_scratch_bytes(n_reqs, num_heads, head_dim, max_ctx_len);
}

extern "C" int rv_paged_attention_decode_static(const void* q, int dtype, int q_stride,
                                                const void* k_cache, const void* v_cache,
                                                const int* block_table, int max_blocks,
                                                const int* ctx_lens, void* out, int n_reqs,
                                                int max_ctx_len, int num_heads, int num_kv_heads,
                                                int head_dim, int page_size, float scale,
                                                int window, void* stream) {
    if (n_reqs == 0) return 0;
    if (n_reqs < 0 || num_heads <= 0 || head_dim <= 0 || max_ctx_len < 0)
        RV_FAIL("paged_attention_decode_static: bad sizes");
    const long long need =
        rv_paged_attention_decode_scratch_bytes(n_reqs, num_heads, head_dim, max_ctx_len);
    if (need > (long long)RV_DECODE_STATIC_SCRATCH_BYTES)
        RV_FAIL("paged_attention_decode_static: %d requests x %d heads x %d tokens x head size %d "
                "need %lld bytes of partial results; the fixed array holds %d. Use "
                "rv_paged_attention_decode with a buffer of your own, or split the batch.",
                n_reqs, num_heads, max_ctx_len, head_dim, need,
                (int)RV_DECODE_STATIC_SCRATCH_BYTES);
    void* scratch = nullptr;
    if (scratch_address(&scratch)) return 1;
    return rv_paged_attention_decode(q, dtype, q_stride, k_cache, v_cache, block_table, max_blocks,
                                     ctx_lens, out, scratch,
                                     (long long)RV_DECODE_STATIC_SCRATCH_BYTES, n_reqs,
                                     max_ctx_len, num_heads, num_kv_heads, head_dim, page_size,
                                     scale, window, stream);
}
