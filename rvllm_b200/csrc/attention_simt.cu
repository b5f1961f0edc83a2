// Paged grouped-query attention in float32 arithmetic on CUDA cores, for float32 or
// bfloat16 storage: the true-32-bit path's attention, and the decode attention of the
// bfloat16 path (decode is bound by reading the pages, not by arithmetic).
//
// Two kernels share the inner loop.
//   paged_attention_warp_kernel    one warp per (token, query head); any number of new
//                                  tokens per request.  Keys are taken 32 at a time in
//                                  groups aligned to absolute position 0, so the order
//                                  of every sum depends on the positions only, not on
//                                  how the tokens were cut into steps.
//   paged_attention_decode_kernel  one block per (request, key/value head, split of 256
//                                  keys); the query heads of a group share each key and
//                                  value load; partial results go to scratch and
//                                  paged_attention_merge_kernel combines the splits in
//                                  order.  Split boundaries are fixed multiples of 256.
//
// A key at position j is visible to the query at position p iff j <= p, and with a
// window iff j > p - window; the softmax is the online form (running maximum and sum).
// Reference counterparts: kv_gather.cu (twice), a batched SGEMM, mask_add_broadcast.cu,
// softmax.cu, a batched SGEMM and transposes (src/cuda/model.rs:528-581).
// Plain reference: tests/plain_ops.py paged_attention.
#include "common.cuh"

#define RV_ATTN_MAX_DPL 8      // head_dim <= 256: up to 8 dimensions per lane
#define RV_ATTN_GT 4           // query heads of a group handled together in decode
#define RV_ATTN_SPLIT 256      // keys per decode split

template <bool kFast>
__device__ __forceinline__ float rv_exp(float x) {
    return kFast ? __expf(x) : expf(x);
}

// dot product of a float32 vector in shared memory with a stored row
__device__ __forceinline__ float rv_dot_row(const float* __restrict__ q, const float* __restrict__ k,
                                            int hd) {
    float s = 0.f;
    for (int d = 0; d < hd; d += 4) {
        const float4 kv = *(const float4*)(k + d);
        s += q[d] * kv.x + q[d + 1] * kv.y + q[d + 2] * kv.z + q[d + 3] * kv.w;
    }
    return s;
}
__device__ __forceinline__ float rv_dot_row(const float* __restrict__ q,
                                            const __nv_bfloat16* __restrict__ k, int hd) {
    float s = 0.f;
    for (int d = 0; d < hd; d += 8) {
        const uint4 raw = *(const uint4*)(k + d);
        const __nv_bfloat162* h = (const __nv_bfloat162*)&raw;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            s += q[d + 2 * i] * f.x + q[d + 2 * i + 1] * f.y;
        }
    }
    return s;
}

// ---------------------------------------------------------------------------------
template <typename T, int DPL>
__global__ void paged_attention_warp_kernel(
    const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache,
    const T* __restrict__ v_cache, const int* __restrict__ block_table, int max_blocks,
    const int* __restrict__ q_start, const int* __restrict__ ctx_lens,
    const int* __restrict__ token_req, T* __restrict__ out, int first_token, int n_tokens,
    int num_heads, int num_kv_heads, int hd, int page_size, float scale, int window) {
    rv_pdl_prologue();
    constexpr bool kFast = sizeof(T) == 2;
    extern __shared__ float q_smem[];   // [warps per block][hd]
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + wib;
    if (warp >= (long long)n_tokens * num_heads) return;
    const int t = first_token + (int)(warp / num_heads);
    const int h = (int)(warp % num_heads);
    const int g = h / (num_heads / num_kv_heads);
    const int r = token_req[t];
    const int clen = ctx_lens[r];
    T* o = out + (size_t)t * num_heads * hd + (size_t)h * hd;
    if (clen == 0) {
        for (int d = lane; d < hd; d += 32) rv_store(o + d, 0.f);
        return;
    }
    const int qs = q_start[r];
    const int p = clen - (q_start[r + 1] - qs) + (t - qs);
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    float* qv = q_smem + wib * hd;
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * hd;
    for (int d = lane; d < hd; d += 32) qv[d] = rv_load(qrow + d);
    __syncwarp();

    float m = -INFINITY, l = 0.f, acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
    const int* table = block_table + (size_t)r * max_blocks;
    const size_t row = (size_t)num_kv_heads * hd;

    for (int base = lo & ~31; base <= p; base += 32) {
        const int j = base + lane;
        const bool valid = j >= lo && j <= p;
        int slot = 0;
        float s = -INFINITY;
        if (valid) {
            slot = table[j / page_size] * page_size + j % page_size;
            s = rv_dot_row(qv, k_cache + (size_t)slot * row + (size_t)g * hd, hd) * scale;
        }
        const float m_new = fmaxf(m, rv_warp_max(s));
        const float pj = valid ? rv_exp<kFast>(s - m_new) : 0.f;
        const float corr = rv_exp<kFast>(m - m_new);
        l = l * corr + rv_warp_sum(pj);
        m = m_new;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[i] *= corr;
        const int count = min(32, p - base + 1);
        for (int jj = 0; jj < count; ++jj) {
            const float pk = __shfl_sync(0xffffffffu, pj, jj);
            const int sk = __shfl_sync(0xffffffffu, slot, jj);
            if (pk != 0.f) {
                const T* vrow = v_cache + (size_t)sk * row + (size_t)g * hd;
#pragma unroll
                for (int i = 0; i < DPL; ++i) {
                    const int d = lane + 32 * i;
                    if (d < hd) acc[i] += pk * rv_load(vrow + d);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) rv_store(o + d, acc[i] / l);
    }
}

// ---------------------------------------------------------------------------------
// Decode: requests [0, n_reqs) bring one token each, token index == request index.
// Scratch per (request, head, split): part_o[hd] (unnormalised) and part_ml = (max, sum).
template <typename T, int DPL>
__global__ void __launch_bounds__(128) paged_attention_decode_kernel(
    const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache,
    const T* __restrict__ v_cache, const int* __restrict__ block_table, int max_blocks,
    const int* __restrict__ ctx_lens, float* __restrict__ part_o, float2* __restrict__ part_ml,
    int max_splits, int num_heads, int num_kv_heads, int hd, int page_size, float scale,
    int window) {
    rv_pdl_prologue();
    constexpr bool kFast = sizeof(T) == 2;
    constexpr int GT = RV_ATTN_GT;
    extern __shared__ float smem[];
    const int G = num_heads / num_kv_heads;
    const int tiles = (G + GT - 1) / GT;
    const int g = blockIdx.x / tiles;                 // key/value head
    const int h0 = g * G + (blockIdx.x % tiles) * GT; // first query head of this block
    const int gcount = min(GT, g * G + G - h0);
    const int r = blockIdx.y;
    const int split = blockIdx.z;
    const int clen = ctx_lens[r];
    if (clen == 0) return;
    const int p = clen - 1;
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    const int k0 = max(lo, split * RV_ATTN_SPLIT);
    const int k1 = min(p, split * RV_ATTN_SPLIT + RV_ATTN_SPLIT - 1);   // inclusive
    if (split < lo / RV_ATTN_SPLIT || k0 > k1) return;

    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    float* qv = smem;                                // [GT][hd]
    float* ps = qv + GT * hd;                        // [4 warps][32][GT]
    int* ss = (int*)(ps + 4 * 32 * GT);              // [4 warps][32]
    float* red = (float*)(ss + 4 * 32);              // [4 warps][GT][hd + 2]
    for (int i = threadIdx.x; i < GT * hd; i += blockDim.x) {
        const int gi = i / hd, d = i - gi * hd;
        qv[i] = gi < gcount ? rv_load(q + (size_t)r * q_stride + (size_t)(h0 + gi) * hd + d) : 0.f;
    }
    __syncthreads();

    float m[GT], l[GT], acc[GT][DPL];
#pragma unroll
    for (int gi = 0; gi < GT; ++gi) {
        m[gi] = -INFINITY;
        l[gi] = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[gi][i] = 0.f;
    }
    const int* table = block_table + (size_t)r * max_blocks;
    const size_t row = (size_t)num_kv_heads * hd;
    float* my_p = ps + w * 32 * GT;
    int* my_s = ss + w * 32;

    const int split_base = split * RV_ATTN_SPLIT;
    for (int base = split_base + w * 32; base <= k1; base += 4 * 32) {
        if (base + 31 < k0) continue;
        const int j = base + lane;
        const bool valid = j >= k0 && j <= k1;
        int slot = 0;
        float s[GT];
#pragma unroll
        for (int gi = 0; gi < GT; ++gi) s[gi] = -INFINITY;
        if (valid) {
            slot = table[j / page_size] * page_size + j % page_size;
            const T* krow = k_cache + (size_t)slot * row + (size_t)g * hd;
#pragma unroll
            for (int gi = 0; gi < GT; ++gi)
                if (gi < gcount) s[gi] = rv_dot_row(qv + gi * hd, krow, hd) * scale;
        }
        my_s[lane] = slot;
#pragma unroll
        for (int gi = 0; gi < GT; ++gi) {
            if (gi < gcount) {
                const float m_new = fmaxf(m[gi], rv_warp_max(s[gi]));
                const float pj = valid ? rv_exp<kFast>(s[gi] - m_new) : 0.f;
                const float corr = rv_exp<kFast>(m[gi] - m_new);
                l[gi] = l[gi] * corr + rv_warp_sum(pj);
                m[gi] = m_new;
#pragma unroll
                for (int i = 0; i < DPL; ++i) acc[gi][i] *= corr;
                my_p[lane * GT + gi] = pj;
            } else {
                my_p[lane * GT + gi] = 0.f;
            }
        }
        __syncwarp();
        const int count = min(32, k1 - base + 1);
        for (int jj = max(0, k0 - base); jj < count; ++jj) {
            const T* vrow = v_cache + (size_t)my_s[jj] * row + (size_t)g * hd;
            float pk[GT];
#pragma unroll
            for (int gi = 0; gi < GT; ++gi) pk[gi] = my_p[jj * GT + gi];
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int d = lane + 32 * i;
                if (d < hd) {
                    const float v = rv_load(vrow + d);
#pragma unroll
                    for (int gi = 0; gi < GT; ++gi) acc[gi][i] += pk[gi] * v;
                }
            }
        }
        __syncwarp();
    }
    // combine the four warps in warp order
    const int rs = hd + 2;
#pragma unroll
    for (int gi = 0; gi < GT; ++gi) {
        float* mine = red + (size_t)(w * GT + gi) * rs;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = lane + 32 * i;
            if (d < hd) mine[d] = acc[gi][i];
        }
        if (lane == 0) {
            mine[hd] = m[gi];
            mine[hd + 1] = l[gi];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < gcount * hd; i += blockDim.x) {
        const int gi = i / hd, d = i - gi * hd;
        float M = -INFINITY;
        for (int ww = 0; ww < 4; ++ww) M = fmaxf(M, red[(size_t)(ww * GT + gi) * rs + hd]);
        float L = 0.f, O = 0.f;
        for (int ww = 0; ww < 4; ++ww) {
            const float* src = red + (size_t)(ww * GT + gi) * rs;
            const float f = src[hd] == -INFINITY ? 0.f : rv_exp<kFast>(src[hd] - M);
            L += src[hd + 1] * f;
            O += src[d] * f;
        }
        const size_t slot = ((size_t)r * num_heads + h0 + gi) * max_splits + split;
        part_o[slot * hd + d] = O;
        if (d == 0) part_ml[slot] = make_float2(M, L);
    }
}

template <typename T>
__global__ void paged_attention_merge_kernel(const float* __restrict__ part_o,
                                             const float2* __restrict__ part_ml,
                                             const int* __restrict__ ctx_lens, T* __restrict__ out,
                                             int max_splits, int num_heads, int hd, int window,
                                             int split_keys) {
    rv_pdl_launch_dependents();
    constexpr bool kFast = sizeof(T) == 2;
    const int r = blockIdx.y, h = blockIdx.x;
    const int clen = ctx_lens[r];                 // the step's index array: before the wait
    rv_pdl_wait();
    T* o = out + ((size_t)r * num_heads + h) * hd;
    if (clen == 0) {
        for (int d = threadIdx.x; d < hd; d += blockDim.x) rv_store(o + d, 0.f);
        return;
    }
    const int p = clen - 1;
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    // A context longer than the launch's max_ctx_len has keys that no split covered: the row
    // is marked invalid (NaN) and nothing outside this head's slots is read.
    if (clen > max_splits * split_keys) {
        for (int d = threadIdx.x; d < hd; d += blockDim.x) rv_store(o + d, NAN);
        return;
    }
    const int s0 = lo / split_keys, s1 = min(p / split_keys, max_splits - 1);
    const size_t base = ((size_t)r * num_heads + h) * max_splits;
    // Splits are combined in order, sixteen at a time: the loads of a group are independent, so
    // a group costs one memory latency, not sixteen.
    constexpr int GROUP = 16;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float M = -INFINITY, L = 0.f, O = 0.f;
        for (int sb = s0; sb <= s1; sb += GROUP) {
            float2 ml[GROUP];
            float po[GROUP];
#pragma unroll
            for (int i = 0; i < GROUP; ++i) {
                const bool valid = sb + i <= s1;
                ml[i] = valid ? part_ml[base + sb + i] : make_float2(-INFINITY, 0.f);
                po[i] = valid ? part_o[(base + sb + i) * hd + d] : 0.f;
            }
            float mg = M;
#pragma unroll
            for (int i = 0; i < GROUP; ++i) mg = fmaxf(mg, ml[i].x);
            if (mg == -INFINITY) continue;
            const float keep = rv_exp<kFast>(M - mg);          // M = -inf -> 0
            O *= keep;
            L *= keep;
#pragma unroll
            for (int i = 0; i < GROUP; ++i) {
                const float w = ml[i].y > 0.f ? rv_exp<kFast>(ml[i].x - mg) : 0.f;
                O += po[i] * w;
                L += ml[i].y * w;
            }
            M = mg;
        }
        rv_store(o + d, L > 0.f ? O / L : 0.f);
    }
}

// ---------------------------------------------------------------------------------
static int check_attention_sizes(const char* name, int num_heads, int num_kv_heads, int hd,
                                 int page_size, int dtype) {
    if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads)
        RV_FAIL("%s: invalid head counts: %d query, %d KV", name, num_heads, num_kv_heads);
    const int step = dtype == RV_DTYPE_BF16 ? 8 : 4;
    if (hd <= 0 || hd % step || hd > 32 * RV_ATTN_MAX_DPL)
        RV_FAIL("%s: head size %d is not supported (a multiple of %d, at most %d)", name, hd, step,
                32 * RV_ATTN_MAX_DPL);
    if (page_size <= 0) RV_FAIL("%s: bad page size %d", name, page_size);
    return 0;
}

#define RV_DISPATCH_DPL(hd, ...)                                          \
    switch (((hd) + 31) / 32) {                                           \
        case 1: { constexpr int DPL = 1; __VA_ARGS__; break; }            \
        case 2: { constexpr int DPL = 2; __VA_ARGS__; break; }            \
        case 3: { constexpr int DPL = 3; __VA_ARGS__; break; }            \
        case 4: { constexpr int DPL = 4; __VA_ARGS__; break; }            \
        case 5: case 6: { constexpr int DPL = 6; __VA_ARGS__; break; }    \
        default: { constexpr int DPL = 8; __VA_ARGS__; break; }           \
    }

extern "C" int rv_paged_attention_warp(const void* q, int dtype, int q_stride, const void* k_cache,
                                       const void* v_cache, const int* block_table, int max_blocks,
                                       const int* q_start, const int* ctx_lens,
                                       const int* token_req, void* out, int first_token,
                                       int n_tokens, int num_heads, int num_kv_heads, int hd,
                                       int page_size, float scale, int window, void* stream) {
    if (n_tokens == 0) return 0;
    if (check_attention_sizes("paged_attention", num_heads, num_kv_heads, hd, page_size, dtype))
        return 1;
    const int wpb = 4;
    const long long warps = (long long)n_tokens * num_heads;
    const long long blocks = (warps + wpb - 1) / wpb;
    if (blocks > 0x7fffffffLL) RV_FAIL("paged_attention: too many rows");
    const size_t smem = (size_t)wpb * hd * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    RV_DISPATCH_DTYPE(dtype, "paged_attention",
        RV_DISPATCH_DPL(hd, (rv_launch(paged_attention_warp_kernel<T, DPL>, dim3((int)blocks), dim3(wpb * 32), smem, s, 
            (const T*)q, q_stride, (const T*)k_cache, (const T*)v_cache, block_table, max_blocks,
            q_start, ctx_lens, token_req, (T*)out, first_token, n_tokens, num_heads, num_kv_heads,
            hd, page_size, scale, window))));
    RV_CHECK_LAUNCH("paged_attention");
    return 0;
}

// Bytes of scratch rv_paged_attention_decode needs: part_o then part_ml.
extern "C" long long rv_paged_attention_decode_scratch_bytes(int n_reqs, int num_heads, int hd,
                                                             int max_ctx_len) {
    const long long splits = (max_ctx_len + RV_ATTN_SPLIT - 1) / RV_ATTN_SPLIT;
    const long long slots = (long long)n_reqs * num_heads * (splits > 0 ? splits : 1);
    return slots * hd * 4 + slots * 8;
}

extern "C" int rv_paged_attention_decode(const void* q, int dtype, int q_stride,
                                         const void* k_cache, const void* v_cache,
                                         const int* block_table, int max_blocks,
                                         const int* ctx_lens, void* out, void* scratch,
                                         long long scratch_bytes, int n_reqs, int max_ctx_len,
                                         int num_heads, int num_kv_heads, int hd, int page_size,
                                         float scale, int window, void* stream) {
    if (n_reqs == 0) return 0;
    if (check_attention_sizes("paged_attention_decode", num_heads, num_kv_heads, hd, page_size,
                              dtype))
        return 1;
    int max_splits = (max_ctx_len + RV_ATTN_SPLIT - 1) / RV_ATTN_SPLIT;
    if (max_splits < 1) max_splits = 1;
    if (rv_paged_attention_decode_scratch_bytes(n_reqs, num_heads, hd, max_ctx_len) > scratch_bytes)
        RV_FAIL("paged_attention_decode: scratch of %lld bytes is too small", scratch_bytes);
    if (n_reqs > 65535 || max_splits > 65535) RV_FAIL("paged_attention_decode: batch too large");
    const size_t slots = (size_t)n_reqs * num_heads * max_splits;
    float* part_o = (float*)scratch;
    float2* part_ml = (float2*)((char*)scratch + slots * hd * 4);
    const int G = num_heads / num_kv_heads;
    const int tiles = (G + RV_ATTN_GT - 1) / RV_ATTN_GT;
    dim3 grid(num_kv_heads * tiles, n_reqs, max_splits);
    const size_t smem = (size_t)(RV_ATTN_GT * hd + 4 * 32 * RV_ATTN_GT + 4 * 32 +
                                 4 * RV_ATTN_GT * (hd + 2)) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    RV_DISPATCH_DTYPE(dtype, "paged_attention_decode",
        RV_DISPATCH_DPL(hd, (rv_launch(paged_attention_decode_kernel<T, DPL>, dim3(grid), dim3(128), smem, s, 
            (const T*)q, q_stride, (const T*)k_cache, (const T*)v_cache, block_table, max_blocks,
            ctx_lens, part_o, part_ml, max_splits, num_heads, num_kv_heads, hd, page_size, scale,
            window))));
    RV_CHECK_LAUNCH("paged_attention_decode");
    dim3 mgrid(num_heads, n_reqs);
    RV_DISPATCH_DTYPE(dtype, "paged_attention_merge",
        (rv_launch(paged_attention_merge_kernel<T>, dim3(mgrid), dim3(hd < 32 ? 32 : (hd > 128 ? 128 : ((hd + 31) / 32) * 32)), 0, s, 
            part_o, part_ml, ctx_lens, (T*)out, max_splits, num_heads, hd, window, RV_ATTN_SPLIT)));
    RV_CHECK_LAUNCH("paged_attention_merge");
    return 0;
}

// The merge step alone, for partial results written by another kernel (attention_mma.cu)
// in the same scratch layout.
extern "C" int rv_paged_attention_merge(const void* scratch, const int* ctx_lens, void* out,
                                        int dtype, int n_reqs, int max_ctx_len, int num_heads,
                                        int hd, int window, int split_keys, void* stream) {
    if (n_reqs == 0) return 0;
    if (split_keys <= 0) RV_FAIL("paged_attention_merge: bad split size");
    int max_splits = (max_ctx_len + split_keys - 1) / split_keys;
    if (max_splits < 1) max_splits = 1;
    if (n_reqs < 0 || n_reqs > 65535 || num_heads <= 0 || hd <= 0)
        RV_FAIL("paged_attention_merge: bad sizes");
    const size_t slots = (size_t)n_reqs * num_heads * max_splits;
    const float* part_o = (const float*)scratch;
    const float2* part_ml = (const float2*)((const char*)scratch + slots * hd * 4);
    dim3 mgrid(num_heads, n_reqs);
    const int threads = hd < 32 ? 32 : (hd > 128 ? 128 : ((hd + 31) / 32) * 32);
    RV_DISPATCH_DTYPE(dtype, "paged_attention_merge",
        (rv_launch(paged_attention_merge_kernel<T>, dim3(mgrid), dim3(threads), 0, (cudaStream_t)stream, 
            part_o, part_ml, ctx_lens, (T*)out, max_splits, num_heads, hd, window, split_keys)));
    RV_CHECK_LAUNCH("paged_attention_merge");
    return 0;
}
