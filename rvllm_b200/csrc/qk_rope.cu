// Per-head RMSNorm of q and k, rotate-half rotation, and the write of k and v into
// the paged cache, in one kernel.  One warp per (token, head) of the fused q|k|v row.
//   q heads: normalised and rotated in place
//   k heads: normalised, rotated, written to the key pages at the token's slot
//   v heads: copied to the value pages at the token's slot
// Reference counterparts: rmsnorm.cu (twice), transpose_axes12.cu (five times), rope.cu
// (twice) and kv_write.cu (src/cuda/model.rs:416-519).  Plain reference:
// tests/plain_ops.py qk_norm_rope_write.
#include "common.cuh"

#define RV_MAX_PAIRS_PER_LANE 4   // head_dim <= 256

template <typename T>
__global__ void qk_norm_rope_write_kernel(
    T* __restrict__ qkv, int row_stride, int n_tokens, int num_heads, int num_kv_heads,
    int head_dim, const float* __restrict__ q_weight, const float* __restrict__ k_weight,
    float eps, const float* __restrict__ cos_table, const float* __restrict__ sin_table,
    const int* __restrict__ positions, const int* __restrict__ slot_mapping,
    T* __restrict__ k_cache, T* __restrict__ v_cache) {
    rv_pdl_prologue();
    const int heads_total = num_heads + 2 * num_kv_heads;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= (long long)n_tokens * heads_total) return;
    const int t = (int)(warp / heads_total);
    const int h = (int)(warp - (long long)t * heads_total);
    const int half = head_dim >> 1;
    T* src = qkv + (size_t)t * row_stride + (size_t)h * head_dim;

    if (h >= num_heads + num_kv_heads) {                     // a value head: copy
        const int slot = slot_mapping[t];
        if (slot < 0) return;
        T* dst = v_cache + ((size_t)slot * num_kv_heads + (h - num_heads - num_kv_heads)) * head_dim;
        for (int d = lane; d < head_dim; d += 32) dst[d] = src[d];
        return;
    }
    const bool is_q = h < num_heads;
    const float* w = is_q ? q_weight : k_weight;
    float a[RV_MAX_PAIRS_PER_LANE], b[RV_MAX_PAIRS_PER_LANE];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < RV_MAX_PAIRS_PER_LANE; ++i) {
        const int p = lane + 32 * i;
        if (p < half) {
            a[i] = rv_load(src + p);
            b[i] = rv_load(src + p + half);
            ss += a[i] * a[i] + b[i] * b[i];
        }
    }
    float rms = 1.f;
    if (w) {
        ss = rv_warp_sum(ss);
        rms = sqrtf(ss / (float)head_dim + eps);
    }
    T* dst = src;
    if (!is_q) {
        const int slot = slot_mapping[t];
        if (slot < 0) return;
        dst = k_cache + ((size_t)slot * num_kv_heads + (h - num_heads)) * head_dim;
    }
    const size_t trow = cos_table ? (size_t)positions[t] * half : 0;
#pragma unroll
    for (int i = 0; i < RV_MAX_PAIRS_PER_LANE; ++i) {
        const int p = lane + 32 * i;
        if (p < half) {
            float x = a[i], y = b[i];
            if (w) {
                x = x / rms * w[p];
                y = y / rms * w[p + half];
            }
            if (cos_table) {
                const float c = cos_table[trow + p], s = sin_table[trow + p];
                const float xr = x * c - y * s, yr = x * s + y * c;
                x = xr;
                y = yr;
            }
            rv_store(dst + p, x);
            rv_store(dst + p + half, y);
        }
    }
}

extern "C" int rv_qk_norm_rope_write(void* qkv, int dtype, int row_stride, int n_tokens,
                                     int num_heads, int num_kv_heads, int head_dim,
                                     const float* q_weight, const float* k_weight, float eps,
                                     const float* cos_table, const float* sin_table,
                                     const int* positions, const int* slot_mapping, void* k_cache,
                                     void* v_cache, void* stream) {
    if (n_tokens == 0) return 0;
    if (n_tokens < 0 || num_heads <= 0 || num_kv_heads < 0 || head_dim <= 0)
        RV_FAIL("qk_norm_rope_write: bad sizes");
    if (head_dim % 2 || head_dim > 64 * RV_MAX_PAIRS_PER_LANE)
        RV_FAIL("qk_norm_rope_write: head size %d is not supported (even, at most %d)", head_dim,
                64 * RV_MAX_PAIRS_PER_LANE);
    if (num_kv_heads > 0 && (!k_cache || !v_cache || !slot_mapping))
        RV_FAIL("qk_norm_rope_write: key/value heads given without a cache to write");
    if ((cos_table == nullptr) != (sin_table == nullptr) || (cos_table && !positions))
        RV_FAIL("qk_norm_rope_write: incomplete rotation table arguments");
    const long long warps = (long long)n_tokens * (num_heads + 2 * num_kv_heads);
    const long long blocks = (warps + 3) / 4;
    if (blocks > 0x7fffffffLL) RV_FAIL("qk_norm_rope_write: too many rows");
    RV_DISPATCH_DTYPE(dtype, "qk_norm_rope_write",
                      (rv_launch(qk_norm_rope_write_kernel<T>, dim3((int)blocks), dim3(128), 0, (cudaStream_t)stream, 
                          (T*)qkv, row_stride, n_tokens, num_heads, num_kv_heads, head_dim,
                          q_weight, k_weight, eps, cos_table, sin_table, positions, slot_mapping,
                          (T*)k_cache, (T*)v_cache)));
    RV_CHECK_LAUNCH("qk_norm_rope_write");
    return 0;
}
