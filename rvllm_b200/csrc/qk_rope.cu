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

// The same for head sizes 16, 32, 64, 128 and 256: a lane owns 8 consecutive dimensions of
// the first half of a head and the 8 it pairs with in the second half (two 16-byte accesses
// for bfloat16), so head_dim / 16 lanes cover a head and a warp covers 32 / (head_dim / 16)
// heads of one token.
__device__ __forceinline__ void rv_load8(const float* p, float (&v)[8]) {
    const float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void rv_load8(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 raw = *(const uint4*)p;
    const __nv_bfloat162* h = (const __nv_bfloat162*)&raw;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void rv_store8(float* p, const float (&v)[8]) {
    *(float4*)p = make_float4(v[0], v[1], v[2], v[3]);
    *(float4*)(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void rv_store8(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 raw;
    __nv_bfloat162* h = (__nv_bfloat162*)&raw;
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *(uint4*)p = raw;
}

template <typename T>
__global__ void qk_norm_rope_write_vec_kernel(
    T* __restrict__ qkv, int row_stride, int n_tokens, int num_heads, int num_kv_heads,
    int head_dim, const float* __restrict__ q_weight, const float* __restrict__ k_weight,
    float eps, const float* __restrict__ cos_table, const float* __restrict__ sin_table,
    const int* __restrict__ positions, const int* __restrict__ slot_mapping,
    T* __restrict__ k_cache, T* __restrict__ v_cache) {
    rv_pdl_launch_dependents();
    const int heads_total = num_heads + 2 * num_kv_heads;
    const int half = head_dim >> 1;
    const int lph = head_dim >> 4;                       // lanes per head
    const int hpw = 32 / lph;                            // heads per warp
    const int groups = (heads_total + hpw - 1) / hpw;    // warps per token
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= (long long)n_tokens * groups) return;
    const int t = (int)(warp / groups);
    const int h = (int)(warp - (long long)t * groups) * hpw + lane / lph;
    const int d0 = (lane % lph) * 8;                      // first of this lane's 8 dimensions
    const bool live = h < heads_total;
    const bool is_v = live && h >= num_heads + num_kv_heads;
    const bool is_q = live && h < num_heads;
    const float* w = is_q ? q_weight : k_weight;
    // what does not depend on the previous kernel comes before the wait for it: the slot, the
    // norm weights and the rotation angles of this token's position
    const int slot = (live && !is_q) ? slot_mapping[t] : 0;
    float wa[8], wb[8], c[8], sn[8];
    const bool normed = live && !is_v && w != nullptr, rotated = live && !is_v && cos_table != nullptr;
    if (normed) {
        rv_load8(w + d0, wa);
        rv_load8(w + half + d0, wb);
    }
    if (rotated) {
        const size_t trow = (size_t)positions[t] * half + d0;
        rv_load8(cos_table + trow, c);
        rv_load8(sin_table + trow, sn);
    }
    rv_pdl_wait();
    float a[8], b[8];
    float ss = 0.f;
    T* src = qkv + (size_t)t * row_stride + (size_t)(live ? h : 0) * head_dim;
    if (live) {
        rv_load8(src + d0, a);
        rv_load8(src + half + d0, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += a[i] * a[i] + b[i] * b[i];
    }
    // sum over the lanes of this head (groups of lph lanes; every lane of the warp takes part)
    for (int o = lph >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (!live) return;
    if (!is_q && slot < 0) return;
    if (is_v) {
        T* dst = v_cache + ((size_t)slot * num_kv_heads + (h - num_heads - num_kv_heads)) * head_dim;
        rv_store8(dst + d0, a);
        rv_store8(dst + half + d0, b);
        return;
    }
    if (normed) {
        const float rms = sqrtf(ss / (float)head_dim + eps);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            a[i] = a[i] / rms * wa[i];
            b[i] = b[i] / rms * wb[i];
        }
    }
    if (rotated) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float xr = a[i] * c[i] - b[i] * sn[i], yr = a[i] * sn[i] + b[i] * c[i];
            a[i] = xr;
            b[i] = yr;
        }
    }
    T* dst = is_q ? src : k_cache + ((size_t)slot * num_kv_heads + (h - num_heads)) * head_dim;
    rv_store8(dst + d0, a);
    rv_store8(dst + half + d0, b);
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
    const bool pow2 = head_dim >= 16 && (head_dim & (head_dim - 1)) == 0;
    const bool aligned = ((uintptr_t)qkv % 16 == 0) && (row_stride % 8 == 0) &&
                         (!k_cache || ((uintptr_t)k_cache % 16 == 0 && (uintptr_t)v_cache % 16 == 0)) &&
                         (!q_weight || (uintptr_t)q_weight % 16 == 0) &&
                         (!k_weight || (uintptr_t)k_weight % 16 == 0) &&
                         (!cos_table || ((uintptr_t)cos_table % 16 == 0 && (uintptr_t)sin_table % 16 == 0));
    if (pow2 && aligned) {
        const int hpw = 32 / (head_dim >> 4);
        const int heads_total = num_heads + 2 * num_kv_heads;
        const long long vwarps = (long long)n_tokens * ((heads_total + hpw - 1) / hpw);
        const long long vblocks = (vwarps + 3) / 4;
        if (vblocks > 0x7fffffffLL) RV_FAIL("qk_norm_rope_write: too many rows");
        RV_DISPATCH_DTYPE(dtype, "qk_norm_rope_write",
                          (rv_launch(qk_norm_rope_write_vec_kernel<T>, dim3((int)vblocks), dim3(128), 0,
                                     (cudaStream_t)stream, (T*)qkv, row_stride, n_tokens, num_heads,
                                     num_kv_heads, head_dim, q_weight, k_weight, eps, cos_table,
                                     sin_table, positions, slot_mapping, (T*)k_cache, (T*)v_cache)));
        RV_CHECK_LAUNCH("qk_norm_rope_write");
        return 0;
    }
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
