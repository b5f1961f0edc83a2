// Paged grouped-query attention on the tensor cores for bfloat16 storage: flash-style
// prefill, and split-KV decode, from one kernel template.  Compiled once per head size
// (-DRV_HD=<multiple of 16, at most 128>), at the first use of a model with that size.
//
// Work layout.  The query rows of one (request, key/value head) are *packed*: row m is
// (token m / G, query head g*G + m % G), G = heads per key/value head, so the G query
// heads that share a key/value head sit side by side in the M dimension of the matrix
// instruction and every key and value tile is read once for all of them.  A block owns
// 16 * NWARPS packed rows and walks the key tiles of 64 keys that those rows can see;
// tiles are aligned to absolute position 0, so the order of every sum depends on
// positions only, not on how the tokens were cut into steps.
//   prefill  NWARPS = 4, the block walks all its tiles and writes the output rows.
//   decode   NWARPS = 1, one token per request; the block walks the tiles of one split of
//            256 keys and writes unnormalised partial results, which
//            paged_attention_merge_kernel (attention_simt.cu) combines in split order.
// Per tile: S = Q K^T (mma.sync m16n8k16, float32 accumulators), mask by comparison,
// online softmax in float32 (base-2 exponentials of scores pre-multiplied by
// scale * log2 e), P rounded to bfloat16, O += P V.  K and V tiles come from the pages
// through the block table with 16-byte cp.async copies into padded shared-memory rows,
// two stages deep; keys past the context or in released pages are zero-filled.
//
// Reference counterparts: kv_gather.cu (twice), a batched SGEMM, mask_add_broadcast.cu,
// softmax.cu, a batched SGEMM and transposes (src/cuda/model.rs:528-581).  Plain
// reference: tests/plain_ops.py paged_attention.
#include <cuda.h>

#include "common.cuh"

#ifndef RV_HD
#error "compile with -DRV_HD=<head size>"
#endif
#if RV_HD % 16 != 0 || RV_HD > 128 || RV_HD < 16
#error "RV_HD must be a multiple of 16 between 16 and 128"
#endif

#define RV_BN 64                 // keys per tile
#define RV_SPLIT 256             // keys per decode split (must match attention_simt.cu)

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zeroed
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0,
                                         unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(unsigned*)&v;
}

// One tile of 64 keys for a warp's 16 packed rows: S = Q K^T, mask, online softmax, O += P V.
// Rows lane/4 ("a") and lane/4 + 8 ("b") of the warp belong to this thread; a key j counts
// for row a iff lo_a <= j <= hi_a.
// Element offset of 16-byte chunk `chunk` of row `row` in a tile: padded rows, or dense
// 128-byte rows whose chunks are XOR-swizzled with the row number as TMA's 128-byte swizzle
// lays them out (the tile must then start on a 1024-byte boundary and HD must be 64).
template <int HD, bool SW>
__device__ __forceinline__ int tile_offset(int row, int chunk) {
    return SW ? row * HD + ((chunk ^ (row & 7)) << 3) : row * (HD + 8) + (chunk << 3);
}

template <int HD, bool SW = false>
__device__ __forceinline__ void attend_tile(const unsigned (&qf)[HD / 16][4], const bf16* kt,
                                            const bf16* vt, int tile_key0, int lane, int lo_a,
                                            int hi_a, int lo_b, int hi_b, float scale_log2,
                                            float& m_a, float& m_b, float& l_a, float& l_b,
                                            float (&o)[HD / 8][4]) {
    constexpr int KSTEPS = HD / 16;
    // S = Q K^T for 16 rows x 64 keys
    float s[RV_BN / 8][4];
#pragma unroll
    for (int i = 0; i < RV_BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
        for (int nb = 0; nb < RV_BN / 16; ++nb) {
            unsigned b[4];
            ldmatrix_x4(b, kt + tile_offset<HD, SW>(nb * 16 + (lane & 7) + (lane >> 4) * 8,
                                                    kk * 2 + ((lane >> 3) & 1)));
            mma_bf16(s[2 * nb], qf[kk], b[0], b[1]);
            mma_bf16(s[2 * nb + 1], qf[kk], b[2], b[3]);
        }
    }
    // mask, scale, running maximum
    const int key0 = tile_key0 + (lane & 3) * 2;
    float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
    for (int i = 0; i < RV_BN / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int key = key0 + i * 8 + e;
            s[i][e] = (key >= lo_a && key <= hi_a) ? s[i][e] * scale_log2 : -INFINITY;
            s[i][2 + e] = (key >= lo_b && key <= hi_b) ? s[i][2 + e] * scale_log2 : -INFINITY;
            mx_a = fmaxf(mx_a, s[i][e]);
            mx_b = fmaxf(mx_b, s[i][2 + e]);
        }
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
    const float off_a = mn_a == -INFINITY ? 0.f : mn_a, off_b = mn_b == -INFINITY ? 0.f : mn_b;
    const float corr_a = exp2f(m_a - off_a), corr_b = exp2f(m_b - off_b);   // m = -inf -> 0
    m_a = mn_a;
    m_b = mn_b;
    l_a *= corr_a;
    l_b *= corr_b;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        o[i][0] *= corr_a; o[i][1] *= corr_a;
        o[i][2] *= corr_b; o[i][3] *= corr_b;
    }
    // P = exp2(S - m), rounded to bfloat16 for the second product; the row sum adds the
    // rounded values, so numerator and denominator see the same numbers
    unsigned pa[RV_BN / 16][4];
#pragma unroll
    for (int i = 0; i < RV_BN / 8; ++i) {
        const float e0 = exp2f(s[i][0] - off_a), e1 = exp2f(s[i][1] - off_a);
        const float e2 = exp2f(s[i][2] - off_b), e3 = exp2f(s[i][3] - off_b);
        const __nv_bfloat162 ra = __floats2bfloat162_rn(e0, e1);
        const __nv_bfloat162 rb = __floats2bfloat162_rn(e2, e3);
        const float2 fa = __bfloat1622float2(ra), fb = __bfloat1622float2(rb);
        l_a += fa.x + fa.y;
        l_b += fb.x + fb.y;
        pa[i >> 1][(i & 1) * 2] = *(const unsigned*)&ra;
        pa[i >> 1][(i & 1) * 2 + 1] = *(const unsigned*)&rb;
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < RV_BN / 16; ++kk) {
#pragma unroll
        for (int nd = 0; nd < HD / 16; ++nd) {
            unsigned b[4];
            ldmatrix_x4_trans(b, vt + tile_offset<HD, SW>(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8,
                                                          nd * 2 + (lane >> 4)));
            mma_bf16(o[2 * nd], pa[kk], b[0], b[1]);
            mma_bf16(o[2 * nd + 1], pa[kk], b[2], b[3]);
        }
    }
}

template <int HD, int NWARPS, bool SPLIT>
__global__ void __launch_bounds__(NWARPS * 32) paged_attention_mma_kernel(
    const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ k_cache,
    const bf16* __restrict__ v_cache, const int* __restrict__ block_table, int max_blocks,
    const int* __restrict__ q_start, const int* __restrict__ ctx_lens, bf16* __restrict__ out,
    float* __restrict__ part_o, float2* __restrict__ part_ml, int max_splits, int first_req,
    int num_heads, int num_kv_heads, int page_size, float scale_log2, int window) {
    rv_pdl_prologue();
    constexpr int BM = 16 * NWARPS;
    constexpr int LD = HD + 8;          // padded row: conflict-free ldmatrix for HD % 16 == 0
    constexpr int CPR = HD / 8;         // 16-byte chunks per row
    constexpr int KSTEPS = HD / 16;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = (bf16*)smem_raw;                         // [BM][LD]
    bf16* Ks = Qs + BM * LD;                            // [2][BN][LD]
    bf16* Vs = Ks + 2 * RV_BN * LD;                     // [2][BN][LD]

    const int G = num_heads / num_kv_heads;
    const int r = first_req + blockIdx.z;
    const int clen = ctx_lens[r];
    if (clen == 0) return;
    const int qs = q_start[r];
    const int qlen = SPLIT ? 1 : q_start[r + 1] - qs;
    const int rows_total = qlen * G;
    int g, tile, split = 0;
    if (SPLIT) {
        const int tiles_per_head = (G + BM - 1) / BM;
        g = blockIdx.y / tiles_per_head;
        tile = blockIdx.y % tiles_per_head;
        split = blockIdx.x;
    } else {
        g = blockIdx.y;
        tile = gridDim.x - 1 - blockIdx.x;              // heaviest (latest) rows first
    }
    const int m0 = tile * BM;
    if (m0 >= rows_total) return;
    const int pos0 = clen - qlen;                        // position of the request's first token here
    const int tok_lo = m0 / G;
    const int tok_hi = min(rows_total - 1, m0 + BM - 1) / G;
    int key_lo = window > 0 ? max(0, pos0 + tok_lo - window + 1) : 0;
    int key_hi = pos0 + tok_hi;                          // inclusive
    if (SPLIT) {
        key_lo = max(key_lo, split * RV_SPLIT);
        key_hi = min(key_hi, split * RV_SPLIT + RV_SPLIT - 1);
        if (key_lo > key_hi) return;
    }
    const int tile_begin = key_lo / RV_BN, tile_end = key_hi / RV_BN;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
    const int* table = block_table + (size_t)r * max_blocks;
    const size_t kv_row = (size_t)num_kv_heads * HD;

    // ---- Q tile -> shared memory (packed rows), zero beyond the last row ----------------
    for (int c = tid; c < BM * CPR; c += NWARPS * 32) {
        const int m = c / CPR, ch = c - m * CPR;
        const int row = m0 + m;
        const bool valid = row < rows_total;
        const int tok = valid ? row / G : 0, hg = valid ? row - tok * G : 0;
        const bf16* src = q + (size_t)(qs + tok) * q_stride + (size_t)(g * G + hg) * HD + ch * 8;
        cp_async_16(Qs + m * LD + ch * 8, src, valid);
    }
    // Each thread copies the same few rows of every tile: ROWS rows, one 16-byte chunk of K
    // and of V each.  The page lookups of a tile are all issued before the first copy, so
    // they overlap instead of forming a chain of dependent loads.
    constexpr int ROWS = RV_BN * CPR / (NWARPS * 32) > 0 ? (RV_BN * CPR + NWARPS * 32 - 1) / (NWARPS * 32) : 1;
    auto load_tile = [&](int t, int stage) {
        bf16* kd = Ks + stage * RV_BN * LD;
        bf16* vd = Vs + stage * RV_BN * LD;
        size_t off[ROWS];
        bool valid[ROWS];
#pragma unroll
        for (int i = 0; i < ROWS; ++i) {
            const int c = tid + i * NWARPS * 32;
            const int row = c / CPR;
            const int j = t * RV_BN + row;
            int page = -1;
            if (c < RV_BN * CPR && j < clen)
                page = table[page_shift >= 0 ? (j >> page_shift) : (j / page_size)];
            valid[i] = page >= 0;
            const int in_page = page_shift >= 0 ? (j & (page_size - 1)) : (j % page_size);
            off[i] = valid[i] ? ((size_t)page * page_size + in_page) * kv_row + (size_t)g * HD +
                                    (c - row * CPR) * 8 : 0;
        }
#pragma unroll
        for (int i = 0; i < ROWS; ++i) {
            const int c = tid + i * NWARPS * 32;
            if (c < RV_BN * CPR) {
                const int row = c / CPR, ch = c - row * CPR;
                cp_async_16(kd + row * LD + ch * 8, k_cache + off[i], valid[i]);
                cp_async_16(vd + row * LD + ch * 8, v_cache + off[i], valid[i]);
            }
        }
    };
    load_tile(tile_begin, 0);
    cp_async_commit();

    // ---- per-thread state: rows lane/4 and lane/4 + 8 of this warp's 16 rows ------------
    const int row_a = m0 + warp * 16 + (lane >> 2), row_b = row_a + 8;
    const bool ok_a = row_a < rows_total, ok_b = row_b < rows_total;
    const int p_a = ok_a ? pos0 + row_a / G : -1, p_b = ok_b ? pos0 + row_b / G : -1;
    int lo_a = window > 0 ? max(0, p_a - window + 1) : 0;
    int lo_b = window > 0 ? max(0, p_b - window + 1) : 0;
    int hi_a = p_a, hi_b = p_b;
    if (SPLIT) {
        lo_a = max(lo_a, key_lo); lo_b = max(lo_b, key_lo);
        hi_a = min(hi_a, key_hi); hi_b = min(hi_b, key_hi);
    }
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    unsigned qf[KSTEPS][4];
    bool q_loaded = false;

    for (int t = tile_begin; t <= tile_end; ++t) {
        const int stage = (t - tile_begin) & 1;
        if (t + 1 <= tile_end) {
            load_tile(t + 1, stage ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (!q_loaded) {
            q_loaded = true;
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk)
                ldmatrix_x4(qf[kk], Qs + (warp * 16 + (lane & 15)) * LD + kk * 16 + (lane >> 4) * 8);
        }
        const bf16* kt = Ks + stage * RV_BN * LD;
        const bf16* vt = Vs + stage * RV_BN * LD;

        attend_tile<HD>(qf, kt, vt, t * RV_BN, lane, lo_a, hi_a, lo_b, hi_b, scale_log2, m_a, m_b, l_a,
                        l_b, o);
        __syncthreads();    // every warp is done with this stage before it is refilled
    }
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);

    const int col = (lane & 3) * 2;
    if (SPLIT) {
        const float ln2 = 0.6931471805599453f;
        if (ok_a) {
            const size_t slot = ((size_t)r * num_heads + g * G + row_a) * max_splits + split;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i)
                *(float2*)(part_o + slot * HD + i * 8 + col) = make_float2(o[i][0], o[i][1]);
            if ((lane & 3) == 0) part_ml[slot] = make_float2(m_a * ln2, l_a);
        }
        if (ok_b) {
            const size_t slot = ((size_t)r * num_heads + g * G + row_b) * max_splits + split;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i)
                *(float2*)(part_o + slot * HD + i * 8 + col) = make_float2(o[i][2], o[i][3]);
            if ((lane & 3) == 0) part_ml[slot] = make_float2(m_b * ln2, l_b);
        }
    } else {
        if (ok_a) {
            const int tok = row_a / G, hg = row_a - tok * G;
            bf16* dst = out + (size_t)(qs + tok) * num_heads * HD + (size_t)(g * G + hg) * HD + col;
            const float inv = 1.f / l_a;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i)
                *(unsigned*)(dst + i * 8) = pack_bf16(o[i][0] * inv, o[i][1] * inv);
        }
        if (ok_b) {
            const int tok = row_b / G, hg = row_b - tok * G;
            bf16* dst = out + (size_t)(qs + tok) * num_heads * HD + (size_t)(g * G + hg) * HD + col;
            const float inv = 1.f / l_b;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i)
                *(unsigned*)(dst + i * 8) = pack_bf16(o[i][2] * inv, o[i][3] * inv);
        }
    }
}

// Decode: one token per request.  A block owns 16 packed rows (the query heads of one
// key/value head) and one split of 256 keys; its four warps take one tile of 64 keys each,
// so all four tiles are in flight at once, and their results are combined in warp order in
// shared memory before the split's partial result is written.
template <int HD, int NW>
__global__ void __launch_bounds__(NW * 32) paged_attention_decode_mma_kernel(
    const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ k_cache,
    const bf16* __restrict__ v_cache, const int* __restrict__ block_table, int max_blocks,
    const int* __restrict__ ctx_lens, float* __restrict__ part_o, float2* __restrict__ part_ml,
    int max_splits, int num_heads, int num_kv_heads, int page_size, float scale_log2, int window) {
    rv_pdl_prologue();
    constexpr int LD = HD + 8;
    constexpr int CPR = HD / 8;
    constexpr int KSTEPS = HD / 16;
    constexpr int TILE = RV_BN * LD;                   // elements of one K or V tile
    constexpr int SPLIT = NW * RV_BN;                  // keys per block
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = (bf16*)smem_raw;                        // [16][LD]
    bf16* KV = Qs + 16 * LD;                           // [NW warps][K tile, V tile]
    const int G = num_heads / num_kv_heads;
    const int r = blockIdx.z;
    const int clen = ctx_lens[r];
    if (clen == 0) return;
    const int tiles_per_head = (G + 15) / 16;
    // the key/value heads of one (request, split) are neighbouring blocks: they run at the same
    // time and together read whole pages, which are contiguous in memory
    const int g = blockIdx.x / tiles_per_head;
    const int m0 = (blockIdx.x % tiles_per_head) * 16;
    const int split = blockIdx.y;
    const int p = clen - 1;
    const int key_lo = max(window > 0 ? max(0, p - window + 1) : 0, split * SPLIT);
    const int key_hi = min(p, split * SPLIT + SPLIT - 1);
    if (key_lo > key_hi) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
    const int* table = block_table + (size_t)r * max_blocks;
    const size_t kv_row = (size_t)num_kv_heads * HD;
    const int rows = min(16, G - m0);

    for (int c = tid; c < 16 * CPR; c += NW * 32) {
        const int m = c / CPR, ch = c - m * CPR;
        const bool valid = m < rows;
        const bf16* src = q + (size_t)r * q_stride + (size_t)(g * G + m0 + (valid ? m : 0)) * HD + ch * 8;
        cp_async_16(Qs + m * LD + ch * 8, src, valid);
    }
    const int t = split * NW + warp;   // this warp's tile
    const bool active = t * RV_BN <= key_hi && t * RV_BN + RV_BN - 1 >= key_lo;
    bf16* kt = KV + warp * 2 * TILE;
    bf16* vt = kt + TILE;
    if (active) {
        constexpr int ROWS = RV_BN * CPR / 32;
        size_t off[ROWS];
        bool valid[ROWS];
#pragma unroll
        for (int i = 0; i < ROWS; ++i) {
            const int c = lane + i * 32;
            const int row = c / CPR;
            const int j = t * RV_BN + row;
            int page = -1;
            if (j < clen) page = table[page_shift >= 0 ? (j >> page_shift) : (j / page_size)];
            valid[i] = page >= 0;
            const int in_page = page_shift >= 0 ? (j & (page_size - 1)) : (j % page_size);
            off[i] = valid[i] ? ((size_t)page * page_size + in_page) * kv_row + (size_t)g * HD +
                                    (c - row * CPR) * 8 : 0;
        }
#pragma unroll
        for (int i = 0; i < ROWS; ++i) {
            const int c = lane + i * 32;
            const int row = c / CPR, ch = c - row * CPR;
            cp_async_16(kt + row * LD + ch * 8, k_cache + off[i], valid[i]);
            cp_async_16(vt + row * LD + ch * 8, v_cache + off[i], valid[i]);
        }
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    const int row_a = m0 + (lane >> 2), row_b = row_a + 8;
    const bool ok_a = row_a < G, ok_b = row_b < G;
    const int lo_a = key_lo, lo_b = key_lo;
    const int hi_a = ok_a ? key_hi : -1, hi_b = ok_b ? key_hi : -1;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    if (active) {
        unsigned qf[KSTEPS][4];
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk)
            ldmatrix_x4(qf[kk], Qs + (lane & 15) * LD + kk * 16 + (lane >> 4) * 8);
        attend_tile<HD>(qf, kt, vt, t * RV_BN, lane, lo_a, hi_a, lo_b, hi_b, scale_log2, m_a, m_b, l_a,
                        l_b, o);
    }
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    __syncthreads();                                    // the tiles are no longer needed

    // park every warp's rows: red[warp][row][HD + 2] float32 over the tile memory
    float* red = (float*)KV;
    constexpr int RS = HD + 2;
    const int col = (lane & 3) * 2;
    {
        float* mine_a = red + ((size_t)warp * 16 + (lane >> 2)) * RS;
        float* mine_b = mine_a + 8 * RS;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            mine_a[i * 8 + col] = o[i][0]; mine_a[i * 8 + col + 1] = o[i][1];
            mine_b[i * 8 + col] = o[i][2]; mine_b[i * 8 + col + 1] = o[i][3];
        }
        if ((lane & 3) == 0) {
            mine_a[HD] = m_a; mine_a[HD + 1] = l_a;
            mine_b[HD] = m_b; mine_b[HD + 1] = l_b;
        }
    }
    __syncthreads();
    const float ln2 = 0.6931471805599453f;
    for (int i = tid; i < rows * HD; i += NW * 32) {
        const int m = i / HD, d = i - m * HD;
        float M = -INFINITY;
        for (int w = 0; w < NW; ++w) M = fmaxf(M, red[((size_t)w * 16 + m) * RS + HD]);
        float L = 0.f, O = 0.f;
        for (int w = 0; w < NW; ++w) {
            const float* src = red + ((size_t)w * 16 + m) * RS;
            const float f = src[HD] == -INFINITY ? 0.f : exp2f(src[HD] - M);
            L += src[HD + 1] * f;
            O += src[d] * f;
        }
        const size_t slot = ((size_t)r * num_heads + g * G + m0 + m) * max_splits + split;
        part_o[slot * HD + d] = O;
        if (d == 0) part_ml[slot] = make_float2(M * ln2, L);
    }
}


#if RV_HD == 64
// ---------------------------------------------------------------------------------
// Decode as a stream (head size 64, pages of 8, 16, 32 or 64 tokens).  One persistent block
// per SM; each of its six warps is a pipeline of its own.  A warp takes work items --
// (request, key/value head, split of 128 or 256 keys) -- round robin, brings the item's key
// and value tiles (64 keys) from the pages into its private ring of two stages with TMA (one
// 3-D tensor copy per page, box [page_size tokens, one head, 64 dims], 128-byte swizzle,
// completion counted on an mbarrier of the stage) and walks them with the online softmax.
// The copy of the next tile -- of the next item, when this one ends -- is in flight while a
// tile is computed, the block table entries and the context length of the item after the one
// being loaded are fetched one item ahead, and its query rows arrive by cp.async; so the warp
// never waits for a chain of dependent loads, and no warp waits for another.  Only tiles
// that hold keys of the item are copied; a page past the context is zero-filled.  Every
// mbarrier wait is bounded (RV_STREAM_WAIT_CYCLES clock cycles); when one runs out the warp
// records code 12 in `status`, waits (bounded) for its copies in flight and leaves.
#define RV_STREAM_WARPS 6
#define RV_STREAM_STAGES 2
#define RV_STREAM_WAIT_CYCLES 400000000ll   // about 0.2 s: far beyond any real wait

__device__ __forceinline__ unsigned st_smem_u32(const void* p) {
    return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void st_mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(st_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void st_mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(st_smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool st_mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(st_smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded by elapsed clock cycles (a poll may itself block for a while inside the hardware).
__device__ __forceinline__ bool st_mbar_wait(unsigned long long* bar, unsigned parity) {
    const long long start = clock64();
    while (true) {
        if (st_mbar_try_wait(bar, parity)) return true;
        if (clock64() - start > RV_STREAM_WAIT_CYCLES) return false;
    }
}
// One page of one key/value head: box [page_size, 1, 64] at (dim 0, head, first slot).
__device__ __forceinline__ void st_tma_page(void* dst, const CUtensorMap* map, int head, int slot0,
                                            unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(st_smem_u32(dst)), "l"((unsigned long long)map), "r"(st_smem_u32(bar)), "r"(0),
          "r"(head), "r"(slot0)
        : "memory");
}

// What the computing side needs to know of an item whose tiles are on their way.
struct StreamMeta {
    int r, g, m0, split, key_lo, key_hi, t_first, t_last;
};

template <int HD>
__global__ void __launch_bounds__(RV_STREAM_WARPS * 32, 1)
paged_attention_decode_stream_kernel(
    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
    const bf16* __restrict__ q, int q_stride, const int* __restrict__ block_table, int max_blocks,
    const int* __restrict__ ctx_lens, float* __restrict__ part_o, float2* __restrict__ part_ml,
    int max_splits, int item_tiles, int num_heads, int num_kv_heads, int page_size,
    float scale_log2, int window, int n_reqs, int* __restrict__ status) {
    rv_pdl_launch_dependents();     // the wait comes after the first look at the block table
    static_assert(HD == 64, "the stream kernel's stages are 128-byte rows");
    constexpr int LD = HD + 8;                                      // query rows stay padded
    constexpr int KSTEPS = HD / 16;
    constexpr int TILE = RV_BN * HD;                                // elements; dense, swizzled
    constexpr int W = RV_STREAM_WARPS, S = RV_STREAM_STAGES;
    extern __shared__ __align__(16) unsigned char smem_raw[];      // aligned by hand below
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    bf16* ring = (bf16*)base;                                       // [W][S][K tile, V tile]
    bf16* q_slots = ring + (size_t)W * S * 2 * TILE;                // [W][2][16][LD]
    __shared__ __align__(8) unsigned long long full_bar[W][S];
    __shared__ StreamMeta meta_q[W][4];

    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int G = num_heads / num_kv_heads;
    const int tiles_per_head = (G + 15) / 16;
    const int heads_tiles = num_kv_heads * tiles_per_head;
    const long long total = (long long)n_reqs * max_splits * heads_tiles;
    const int nb = gridDim.x, b = blockIdx.x;
    const int page_shift = 31 - __clz(page_size);                   // a power of two (host check)
    const int ppt = RV_BN >> page_shift;                            // pages per tile
    const int ppi = ppt * item_tiles;                               // pages per item (<= 32)
    const int item_keys = item_tiles * RV_BN;
    const unsigned page_bytes = (unsigned)page_size * HD * 2u;

    if (lane == 0) {
        for (int s = 0; s < S; ++s) st_mbar_init(&full_bar[w][s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    bf16* my_ring = ring + (size_t)w * S * 2 * TILE;
    bf16* my_q = q_slots + (size_t)w * 2 * 16 * LD;
    const float ln2 = 0.6931471805599453f;

    // ---- the loading side -----------------------------------------------------------------
    long long lk = 0;                 // this warp's next item is number (lk * W + w) * nb + b
    int n_live = 0;                   // items with keys met so far (index into meta_q and my_q)
    bool l_more = true;               // items left to look at
    int l_t = 0, l_last = -1, l_t0 = 0, l_g = 0, l_page = -1;
    int nx_clen = 0, nx_page = -1;    // context length and this lane's page of item lk, fetched ahead
    // fetch the length and the block table entries of item `it` (no use of them yet)
    auto fetch_ahead = [&](long long it) {
        nx_clen = 0;
        nx_page = -1;
        if (it >= total) return;
        const long long rest = it / heads_tiles;
        const int split = (int)(rest % max_splits), r = (int)(rest / max_splits);
        nx_clen = ctx_lens[r];
        const int blk = ((split * item_keys) >> page_shift) + lane;
        if (lane < ppi && blk < max_blocks) nx_page = block_table[(size_t)r * max_blocks + blk];
    };
    fetch_ahead((lk * W + w) * nb + b);   // index arrays of the step: not the previous kernel's
    rv_pdl_wait();                         // keys, values and queries are the previous kernels'
    int n_loaded = 0, n_consumed = 0;

    // move to the next item that has keys; false when there is none
    auto next_load_item = [&]() -> bool {
        while (l_more) {
            const long long it = (lk * W + w) * nb + b;
            if (it >= total) {
                l_more = false;
                break;
            }
            const int clen = nx_clen, page = nx_page;
            ++lk;
            fetch_ahead((lk * W + w) * nb + b);
            const int ht = (int)(it % heads_tiles);
            const long long rest = it / heads_tiles;
            const int split = (int)(rest % max_splits), r = (int)(rest / max_splits);
            if (clen == 0) continue;
            const int p = clen - 1;
            const int key_lo = max(window > 0 ? max(0, p - window + 1) : 0, split * item_keys);
            const int key_hi = min(p, split * item_keys + item_keys - 1);
            if (key_lo > key_hi) continue;
            const int g = ht / tiles_per_head, m0 = (ht % tiles_per_head) * 16;
            l_g = g;
            l_t0 = split * item_tiles;
            l_t = key_lo / RV_BN;
            l_last = key_hi / RV_BN;
            l_page = (lane < ppi && ((split * item_keys + (lane << page_shift)) < clen)) ? page : -1;
            if (lane == 0) {
                StreamMeta& m = meta_q[w][n_live & 3];
                m.r = r; m.g = g; m.m0 = m0; m.split = split;
                m.key_lo = key_lo; m.key_hi = key_hi; m.t_first = l_t; m.t_last = l_last;
            }
            // its query rows, by cp.async into the slot of this item's parity
            bf16* Qs = my_q + (size_t)(n_live & 1) * 16 * LD;
            const int rows = min(16, G - m0);
            for (int i = lane; i < 16 * (HD / 8); i += 32) {
                const int m = i / (HD / 8), ch = i - m * (HD / 8);
                const bool valid = m < rows;
                const bf16* src = q + (size_t)r * q_stride +
                                  (size_t)(g * G + m0 + (valid ? m : 0)) * HD + ch * 8;
                cp_async_16(Qs + m * LD + ch * 8, src, valid);
            }
            cp_async_commit();
            ++n_live;
            __syncwarp();
            return true;
        }
        return false;
    };
    // copy the load cursor's tile into the next stage; the stage is free (the caller knows)
    auto issue_tile = [&]() {
        const int s = n_loaded % S;
        bf16* kd = my_ring + (size_t)s * 2 * TILE;
        bf16* vd = kd + TILE;
        unsigned long long* bar = &full_bar[w][s];
        const int src = (l_t - l_t0) * ppt + lane;
        const int page = __shfl_sync(0xffffffffu, l_page, src & 31);
        const bool mine = lane < ppt;
        const unsigned have = __ballot_sync(0xffffffffu, mine && page >= 0);
        const unsigned miss = __ballot_sync(0xffffffffu, mine && page < 0);
        if (miss) {                                 // pages past the context read as zeros
            const uint4 z = make_uint4(0, 0, 0, 0);
            for (int pi = 0; pi < ppt; ++pi) {
                if (!((miss >> pi) & 1u)) continue;
                uint4* kz = (uint4*)(kd + (size_t)pi * page_size * HD);
                uint4* vz = (uint4*)(vd + (size_t)pi * page_size * HD);
                for (int i = lane; i < (int)(page_bytes / 16); i += 32) {
                    kz[i] = z;
                    vz[i] = z;
                }
            }
        }
        // the stage's earlier reads (ldmatrix) and the zeros above come before the copies
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) st_mbar_expect_tx(bar, (unsigned)__popc(have) * 2u * page_bytes);
        __syncwarp();
        if (mine && page >= 0) {
            st_tma_page(kd + (size_t)lane * page_size * HD, &map_k, l_g, page << page_shift, bar);
            st_tma_page(vd + (size_t)lane * page_size * HD, &map_v, l_g, page << page_shift, bar);
        }
        ++n_loaded;
        ++l_t;
    };
    auto fill = [&]() {
        while (n_loaded - n_consumed < S) {
            if (l_t > l_last && !next_load_item()) break;
            issue_tile();
        }
    };

    // ---- the computing side -----------------------------------------------------------------
    fill();
    int n_done = 0;                   // items finished (index into meta_q and my_q)
    bool failed = false;
    while (n_consumed < n_loaded && !failed) {
        __syncwarp();
        const StreamMeta m = meta_q[w][n_done & 3];
        const int rows = min(16, G - m.m0);
        unsigned qf[KSTEPS][4];
        {
            cp_async_wait<0>();
            __syncwarp();
            const bf16* Qs = my_q + (size_t)(n_done & 1) * 16 * LD;
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk)
                ldmatrix_x4(qf[kk], Qs + (lane & 15) * LD + kk * 16 + (lane >> 4) * 8);
            __syncwarp();
        }
        const int row_a = m.m0 + (lane >> 2), row_b = row_a + 8;
        const bool ok_a = (lane >> 2) < rows, ok_b = (lane >> 2) + 8 < rows;
        const int hi_a = ok_a ? m.key_hi : -1, hi_b = ok_b ? m.key_hi : -1;
        float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
        float o[HD / 8][4];
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
        for (int t = m.t_first; t <= m.t_last; ++t) {
            const int s = n_consumed % S;
            if (!st_mbar_wait(&full_bar[w][s], (unsigned)(n_consumed / S) & 1u)) {
                failed = true;
                break;
            }
            const bf16* kt = my_ring + (size_t)s * 2 * TILE;
            attend_tile<HD, true>(qf, kt, kt + TILE, t * RV_BN, lane, m.key_lo, hi_a, m.key_lo, hi_b,
                                  scale_log2, m_a, m_b, l_a, l_b, o);
            __syncwarp();
            ++n_consumed;
            fill();                                 // the freed stage takes the next tile
        }
        if (failed) break;
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
        const int col = (lane & 3) * 2;
        if (ok_a) {
            const size_t slot = ((size_t)m.r * num_heads + m.g * G + row_a) * max_splits + m.split;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i)
                *(float2*)(part_o + slot * HD + i * 8 + col) = make_float2(o[i][0], o[i][1]);
            if ((lane & 3) == 0) part_ml[slot] = make_float2(m_a * ln2, l_a);
        }
        if (ok_b) {
            const size_t slot = ((size_t)m.r * num_heads + m.g * G + row_b) * max_splits + m.split;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i)
                *(float2*)(part_o + slot * HD + i * 8 + col) = make_float2(o[i][2], o[i][3]);
            if ((lane & 3) == 0) part_ml[slot] = make_float2(m_b * ln2, l_b);
        }
        ++n_done;
    }
    if (failed) {
        // record it, then wait (bounded) for the copies that are still on their way: none may
        // arrive after the block has left
        if (lane == 0) atomicCAS(status, 0, 12);
        const long long start = clock64();
        for (int i = n_consumed; i < n_loaded; ++i) {
            bool done = false;
            while (!done && clock64() - start < RV_STREAM_WAIT_CYCLES)
                done = st_mbar_try_wait(&full_bar[w][i % S], (unsigned)(i / S) & 1u);
        }
        cp_async_wait<0>();
    }
}
#endif

static thread_local char g_error[512] = "";
static int fail(const char* msg) {
    snprintf(g_error, sizeof(g_error), "%s", msg);
    return 1;
}
#define RV_CAT2(a, b) a##b
#define RV_CAT(a, b) RV_CAT2(a, b)
#define RV_SYM(name) RV_CAT(RV_CAT(name, _hd), RV_HD)

extern "C" const char* RV_SYM(rv_attention_mma_last_error)() { return g_error; }

template <int NWARPS>
static size_t smem_bytes() {
    return (size_t)(16 * NWARPS + 4 * RV_BN) * (RV_HD + 8) * sizeof(bf16);
}

// Prefill: requests [first_req, first_req + n_reqs), the longest bringing max_q_len tokens.
extern "C" int RV_SYM(rv_paged_attention_prefill_mma)(
    const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* block_table,
    int max_blocks, const int* q_start, const int* ctx_lens, void* out, int first_req, int n_reqs,
    int max_q_len, int num_heads, int num_kv_heads, int page_size, float scale, int window,
    void* stream) {
    if (n_reqs == 0) return 0;
    if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads || page_size <= 0 ||
        max_q_len <= 0 || n_reqs < 0)
        return fail("paged_attention_prefill_mma: bad sizes");
    const int G = num_heads / num_kv_heads;
    const long long tiles = ((long long)max_q_len * G + 63) / 64;
    if (tiles > 0x7fffffffLL || num_kv_heads > 65535 || n_reqs > 65535)
        return fail("paged_attention_prefill_mma: batch too large for one launch");
    // 4 warps (64 packed rows per block) by default.  8 warps reuse every key and value tile
    // for twice as many rows but measured slower at 2,048 tokens (138.5 against 126.7 us per
    // layer at LFM2-1.2B sizes); RVLLM_ATTN_PREFILL_WARPS=8 selects them.
    static int warps = -1;
    if (warps < 0) {
        const char* e = getenv("RVLLM_ATTN_PREFILL_WARPS");
        warps = (e && atoi(e) == 8) ? 8 : 4;
        const size_t big = smem_bytes<8>();
        cudaError_t err = cudaSuccess;
        if (big > 48 * 1024) {
            err = cudaFuncSetAttribute(paged_attention_mma_kernel<RV_HD, 8, false>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)big);
            if (err == cudaSuccess && smem_bytes<4>() > 48 * 1024)
                err = cudaFuncSetAttribute(paged_attention_mma_kernel<RV_HD, 4, false>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)smem_bytes<4>());
        }
        if (err != cudaSuccess) { warps = -1; return fail(cudaGetErrorString(err)); }
    }
    const int rows_per_block = 16 * warps;
    const long long blocks_x = ((long long)max_q_len * G + rows_per_block - 1) / rows_per_block;
    dim3 grid((unsigned)blocks_x, num_kv_heads, n_reqs);
    if (warps == 8)
        rv_launch(paged_attention_mma_kernel<RV_HD, 8, false>, dim3(grid), dim3(256), smem_bytes<8>(),
                  (cudaStream_t)stream, (const bf16*)q, q_stride, (const bf16*)k_cache,
                  (const bf16*)v_cache, block_table, max_blocks, q_start, ctx_lens, (bf16*)out,
                  (float*)nullptr, (float2*)nullptr, 0, first_req, num_heads, num_kv_heads, page_size,
                  scale * 1.4426950408889634f, window);
    else
        rv_launch(paged_attention_mma_kernel<RV_HD, 4, false>, dim3(grid), dim3(128), smem_bytes<4>(),
                  (cudaStream_t)stream, (const bf16*)q, q_stride, (const bf16*)k_cache,
                  (const bf16*)v_cache, block_table, max_blocks, q_start, ctx_lens, (bf16*)out,
                  (float*)nullptr, (float2*)nullptr, 0, first_req, num_heads, num_kv_heads, page_size,
                  scale * 1.4426950408889634f, window);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(cudaGetErrorString(e));
    return 0;
}

// Decode: requests [0, n_reqs) bring one token each (token index == request index).
// Writes partial results for paged_attention_merge_kernel; scratch layout as in
// rv_paged_attention_decode: part_o [n_reqs * heads * max_splits][HD], then part_ml.
extern "C" int RV_SYM(rv_paged_attention_decode_mma)(
    const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* block_table,
    int max_blocks, const int* q_start, const int* ctx_lens, void* scratch, long long scratch_bytes,
    int n_reqs, int max_ctx_len, int num_heads, int num_kv_heads, int page_size, float scale,
    int window, int split_keys, void* stream) {
    if (n_reqs == 0) return 0;
    if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads || page_size <= 0 ||
        n_reqs < 0)
        return fail("paged_attention_decode_mma: bad sizes");
    if (split_keys != 128 && split_keys != 256)
        return fail("paged_attention_decode_mma: the split is 128 or 256 keys");
    int max_splits = (max_ctx_len + split_keys - 1) / split_keys;
    if (max_splits < 1) max_splits = 1;
    const size_t slots = (size_t)n_reqs * num_heads * max_splits;
    if ((long long)(slots * RV_HD * 4 + slots * 8) > scratch_bytes)
        return fail("paged_attention_decode_mma: scratch too small");
    const int G = num_heads / num_kv_heads;
    const int tiles_per_head = (G + 15) / 16;
    if (n_reqs > 65535 || num_kv_heads * tiles_per_head > 65535)
        return fail("paged_attention_decode_mma: batch too large for one launch");
    static bool configured = false;
    const size_t smem4 = (size_t)(16 + 8 * RV_BN) * (RV_HD + 8) * sizeof(bf16);
    const size_t smem2 = (size_t)(16 + 4 * RV_BN) * (RV_HD + 8) * sizeof(bf16);
    if (!configured) {
        cudaError_t e = cudaSuccess;
        if (smem4 > 48 * 1024)
            e = cudaFuncSetAttribute(paged_attention_decode_mma_kernel<RV_HD, 4>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem4);
        if (e == cudaSuccess && smem2 > 48 * 1024)
            e = cudaFuncSetAttribute(paged_attention_decode_mma_kernel<RV_HD, 2>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
        if (e != cudaSuccess) return fail(cudaGetErrorString(e));
        configured = true;
    }
    if (max_splits > 65535) return fail("paged_attention_decode_mma: context too long for one launch");
    dim3 grid(num_kv_heads * tiles_per_head, max_splits, n_reqs);
    float* part_o = (float*)scratch;
    float2* part_ml = (float2*)((char*)scratch + slots * RV_HD * 4);
    if (split_keys == 256)
        rv_launch(paged_attention_decode_mma_kernel<RV_HD, 4>, dim3(grid), dim3(128), smem4,
                  (cudaStream_t)stream, (const bf16*)q, q_stride, (const bf16*)k_cache,
                  (const bf16*)v_cache, block_table, max_blocks, ctx_lens, part_o, part_ml,
                  max_splits, num_heads, num_kv_heads, page_size, scale * 1.4426950408889634f, window);
    else
        rv_launch(paged_attention_decode_mma_kernel<RV_HD, 2>, dim3(grid), dim3(64), smem2,
                  (cudaStream_t)stream, (const bf16*)q, q_stride, (const bf16*)k_cache,
                  (const bf16*)v_cache, block_table, max_blocks, ctx_lens, part_o, part_ml,
                  max_splits, num_heads, num_kv_heads, page_size, scale * 1.4426950408889634f, window);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(cudaGetErrorString(e));
    return 0;
}

// Decode as a stream (one persistent block per SM); same scratch layout as
// rv_paged_attention_decode_mma with the split that rv_paged_attention_decode_stream_split
// names (128 or 256 keys: the smaller one when the larger would leave warps without work).
// Needs head size 64 and pages of 8, 16, 32 or 64 tokens; `total_slots` = pages * page_size
// of the cache tensors.  `status` receives code 12 when a bounded wait runs out.
#if RV_HD == 64
typedef CUresult (*RvEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int kv_map(CUtensorMap* map, const void* cache, long long total_slots, int num_kv_heads,
                  int page_size) {
    static RvEncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) !=
                cudaSuccess || qr != cudaDriverEntryPointSuccess)
            return fail("paged_attention_decode_stream: cuTensorMapEncodeTiled is not available");
        fn = (RvEncodeTiledFn)p;
    }
    cuuint64_t dims[3] = {RV_HD, (cuuint64_t)num_kv_heads, (cuuint64_t)total_slots};
    cuuint64_t strides[2] = {RV_HD * 2, (cuuint64_t)num_kv_heads * RV_HD * 2};
    cuuint32_t box[3] = {RV_HD, 1, (cuuint32_t)page_size};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(cache), dims, strides,
                    box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("paged_attention_decode_stream: cuTensorMapEncodeTiled failed");
    return 0;
}

extern "C" int RV_SYM(rv_paged_attention_decode_stream_split)(int n_reqs, int max_ctx_len,
                                                              int num_heads, int num_kv_heads,
                                                              int n_sms) {
    if (num_kv_heads <= 0 || n_sms <= 0) return RV_SPLIT;
    const int G = num_heads / num_kv_heads;
    const long long items = (long long)n_reqs * ((max_ctx_len + RV_SPLIT - 1) / RV_SPLIT) *
                            num_kv_heads * ((G + 15) / 16);
    return items < 3ll * RV_STREAM_WARPS * n_sms ? RV_SPLIT / 2 : RV_SPLIT;
}

extern "C" int RV_SYM(rv_paged_attention_decode_stream)(
    const void* q, int q_stride, const void* k_cache, const void* v_cache, long long total_slots,
    const int* block_table, int max_blocks, const int* ctx_lens, void* scratch,
    long long scratch_bytes, int n_reqs, int max_ctx_len, int num_heads, int num_kv_heads,
    int page_size, float scale, int window, int split_keys, int n_sms, int* status, void* stream) {
    if (n_reqs == 0) return 0;
    if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads || n_reqs < 0 || n_sms <= 0)
        return fail("paged_attention_decode_stream: bad sizes");
    if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64)
        return fail("paged_attention_decode_stream: pages of 8, 16, 32 or 64 tokens only");
    if (split_keys != RV_SPLIT && split_keys != RV_SPLIT / 2)
        return fail("paged_attention_decode_stream: splits of 128 or 256 keys only");
    if (((uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)q) % 16 || (q_stride % 8))
        return fail("paged_attention_decode_stream: caches and query rows must be 16-byte aligned");
    int max_splits = (max_ctx_len + split_keys - 1) / split_keys;
    if (max_splits < 1) max_splits = 1;
    const size_t slots = (size_t)n_reqs * num_heads * max_splits;
    if ((long long)(slots * RV_HD * 4 + slots * 8) > scratch_bytes)
        return fail("paged_attention_decode_stream: scratch too small");
    const int G = num_heads / num_kv_heads;
    const int tiles_per_head = (G + 15) / 16;
    const long long total = (long long)n_reqs * max_splits * num_kv_heads * tiles_per_head;
    const size_t ring_bytes = (size_t)RV_STREAM_WARPS * RV_STREAM_STAGES * 2 * RV_BN * RV_HD * sizeof(bf16);
    const size_t q_bytes = (size_t)RV_STREAM_WARPS * 2 * 16 * (RV_HD + 8) * sizeof(bf16);
    const size_t smem = ring_bytes + q_bytes + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(paged_attention_decode_stream_kernel<RV_HD>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(cudaGetErrorString(e));
        configured = true;
    }
    CUtensorMap map_k, map_v;
    if (kv_map(&map_k, k_cache, total_slots, num_kv_heads, page_size)) return 1;
    if (kv_map(&map_v, v_cache, total_slots, num_kv_heads, page_size)) return 1;
    long long blocks = (total + RV_STREAM_WARPS - 1) / RV_STREAM_WARPS;
    if (blocks > n_sms) blocks = n_sms;
    float* part_o = (float*)scratch;
    float2* part_ml = (float2*)((char*)scratch + slots * RV_HD * 4);
    rv_launch(paged_attention_decode_stream_kernel<RV_HD>, dim3((unsigned)blocks),
              dim3(RV_STREAM_WARPS * 32), smem, (cudaStream_t)stream, map_k, map_v,
              (const bf16*)q, q_stride, block_table, max_blocks, ctx_lens, part_o, part_ml,
              max_splits, split_keys / RV_BN, num_heads, num_kv_heads, page_size,
              scale * 1.4426950408889634f, window, n_reqs, status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(cudaGetErrorString(e));
    return 0;
}
#endif
