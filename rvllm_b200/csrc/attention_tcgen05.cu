// Paged causal attention for prompt portions on the 5th-generation tensor cores (bfloat16,
// head size 64, pages of 8 to 64 tokens).
//
// One block per (request, key/value head, block of query tokens).  The block's 128 rows are
// its query tokens times the G query heads that share the key/value head (row = token * G +
// head), so one key/value tile serves all of them.  Per tile of 64 keys:
//   S = Q K^T     tcgen05.mma (M = 128, N = 64, four K = 16 steps), Q and K in shared memory
//                 (K-major, 128-byte swizzle), S in TMEM columns [0, 64);
//   softmax       each of 128 threads owns one row: it reads its S row from TMEM
//                 (tcgen05.ld), masks where the tile needs it, keeps the running maximum and
//                 sum in float32, rescales its O row in TMEM (tcgen05.ld / tcgen05.st, only
//                 when a maximum of its warp moved) and writes P as bfloat16 into a swizzled
//                 shared-memory tile -- no shuffles, no shared-memory reductions;
//   O += P V      tcgen05.mma (M = 128, N = 64, four K = 16 steps), P from shared memory
//                 (K-major), V as it lies in the cache ([key][dim], i.e. MN-major), O in TMEM
//                 columns [64, 128).
// 65 KB of shared memory and 128 TMEM columns per block: three blocks share an SM, so one
// block's softmax overlaps the others' copies and MMAs.  The exponent's offset follows the
// row maximum lazily (it moves only when the maximum has grown by more than 2^8), so O is
// rescaled on few tiles.
//
// Roles: warps 0-3 are the 128 rows; warp 4 brings Q (one 3-D TMA copy: [tokens, heads, 64])
// and the key and value tiles (one 3-D TMA copy per page) into rings of two stages, keys and
// values each as soon as their stage is free; thread 0 of warp 5 issues the MMAs -- S of the
// next tile as soon as every row has read the current S out of TMEM.  Roles that wait do not
// share a warp: a spinning lane starves the other lanes of its warp.  Only mbarriers
// synchronise the roles inside the loop ("keys arrived", "values arrived", "S ready", "S
// read", "P written", "P V done", "stage free").  Every mbarrier wait is bounded in clock
// cycles; when one runs out the block records code 21 in `status`, the roles walk their
// remaining tiles without issuing anything (so every arrival still happens), the producer
// waits (bounded) for its copies in flight, TMEM is freed and the block returns.
//
// Reference counterparts: kv_gather.cu (twice), a batched SGEMM, mask_add_broadcast.cu,
// softmax.cu, a batched SGEMM and transposes (src/cuda/model.rs:528-581).  Plain reference:
// tests/plain_ops.py paged_attention.
#include <cuda.h>

#include "common.cuh"

#ifndef RV_HD
#define RV_HD 64
#endif
#define AT_ROWS 128
#define AT_KEYS 64
#define AT_STAGES 2
#define AT_WAIT_CYCLES 400000000ll       // about 0.2 s: far beyond any real wait

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ unsigned at_smem(const void* p) {
    return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void at_mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(at_smem(bar)), "r"(count));
}
__device__ __forceinline__ void at_mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(at_smem(bar)) : "memory");
}
__device__ __forceinline__ void at_mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(at_smem(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool at_mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(at_smem(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
__device__ __forceinline__ bool at_mbar_wait(unsigned long long* bar, unsigned parity,
                                             volatile int* failed) {
    if (at_mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    for (unsigned i = 1;; ++i) {
        if (at_mbar_try_wait(bar, parity)) return true;
        if (*failed) return false;
        if ((i & 63u) == 0 && clock64() - start > AT_WAIT_CYCLES) return false;
    }
}
__device__ __forceinline__ void at_tma_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2,
                                          unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(at_smem(dst)), "l"((unsigned long long)map), "r"(at_smem(bar)), "r"(c0), "r"(c1),
          "r"(c2)
        : "memory");
}
__device__ __forceinline__ void at_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(at_smem(bar))
                 : "memory");
}
__device__ __forceinline__ void at_mma(unsigned tmem_d, unsigned long long a_desc,
                                       unsigned long long b_desc, unsigned idesc,
                                       unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void at_tmem_ld16(unsigned taddr, float (&r)[16]) {
    unsigned u[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, "
        "%12, %13, %14, %15}, [%16];"
        : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]),
          "=r"(u[7]), "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]),
          "=r"(u[14]), "=r"(u[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) r[i] = __uint_as_float(u[i]);
}
// A whole row of 64 columns in one instruction, and the wait for it in the same statement,
// so that no use of the values can be scheduled before the wait.
__device__ __forceinline__ void at_tmem_ld64(unsigned taddr, float (&r)[64]) {
    unsigned u[64];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]), "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]), "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31]), "=r"(u[32]), "=r"(u[33]), "=r"(u[34]), "=r"(u[35]), "=r"(u[36]), "=r"(u[37]), "=r"(u[38]), "=r"(u[39]), "=r"(u[40]), "=r"(u[41]), "=r"(u[42]), "=r"(u[43]), "=r"(u[44]), "=r"(u[45]), "=r"(u[46]), "=r"(u[47]), "=r"(u[48]), "=r"(u[49]), "=r"(u[50]), "=r"(u[51]), "=r"(u[52]), "=r"(u[53]), "=r"(u[54]), "=r"(u[55]), "=r"(u[56]), "=r"(u[57]), "=r"(u[58]), "=r"(u[59]), "=r"(u[60]), "=r"(u[61]), "=r"(u[62]), "=r"(u[63])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 64; ++i) r[i] = __uint_as_float(u[i]);
}
__device__ __forceinline__ float at_exp2(float x) {           // 2^x, flushing; -inf -> 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void at_tmem_st16(unsigned taddr, const float (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, "
        "%12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(__float_as_uint(r[0])), "r"(__float_as_uint(r[1])),
          "r"(__float_as_uint(r[2])), "r"(__float_as_uint(r[3])), "r"(__float_as_uint(r[4])),
          "r"(__float_as_uint(r[5])), "r"(__float_as_uint(r[6])), "r"(__float_as_uint(r[7])),
          "r"(__float_as_uint(r[8])), "r"(__float_as_uint(r[9])), "r"(__float_as_uint(r[10])),
          "r"(__float_as_uint(r[11])), "r"(__float_as_uint(r[12])), "r"(__float_as_uint(r[13])),
          "r"(__float_as_uint(r[14])), "r"(__float_as_uint(r[15]))
        : "memory");
}
// Shared-memory matrix descriptor, 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024
// bytes apart (stride byte offset 64 x 16), descriptor version 1, layout type 2.  The same
// form serves a K-major operand (rows = M or N index, 64 K elements per row) and an MN-major
// one (rows = K index, 64 M or N elements per row).
__device__ __forceinline__ unsigned long long at_desc(const void* tile) {
    const unsigned long long addr = (at_smem(tile) & 0x3FFFFu) >> 4;
    return addr | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

template <int HD>
__global__ void __launch_bounds__(192, 3) paged_attention_prefill_tcgen05_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table, int max_blocks,
    const int* __restrict__ q_start, const int* __restrict__ ctx_lens, bf16* __restrict__ out,
    int first_req, int num_heads, int num_kv_heads, int q_block, int page_size, float scale_log2,
    int window, int* __restrict__ status, int nsplit, float* __restrict__ part_o,
    float2* __restrict__ part_ml) {
    static_assert(HD == 64, "one 128-byte swizzle row per key");
    rv_pdl_prologue();
    // blocks are handed out in the order x, then y: with the key/value head in x, all heads of a
    // request's longest block of query tokens start first, then all heads of the next longest
    // nsplit > 1: the key tiles of a block of query tokens are shared out over `nsplit` blocks
    // (blockIdx.z = request * nsplit + part), each leaving its unnormalised O rows, offsets and
    // sums in `part_o` / `part_ml` for paged_attention_prefill_merge_kernel
    const int r_local = (int)blockIdx.z / nsplit, part = (int)blockIdx.z - r_local * nsplit;
    const int r = first_req + r_local, g = blockIdx.x;
    const int clen = ctx_lens[r];
    const int qs = q_start[r];
    const int qlen = q_start[r + 1] - qs;
    const int nqb = (qlen + q_block - 1) / q_block;
    if ((int)blockIdx.y >= nqb || clen == 0) return;           // the whole block, before any set-up
    const int qb = nqb - 1 - blockIdx.y;                        // the longest blocks start first
    const int G = num_heads / num_kv_heads;
    const int q0 = qb * q_block;
    const int n_tok = min(q_block, qlen - q0);                  // query tokens of this block
    const int start = clen - qlen;                              // position of the portion's first token
    const int p_first = start + q0, p_last = p_first + n_tok - 1;
    const int key_lo = window > 0 ? max(0, p_first - window + 1) : 0;
    const int t_all = key_lo / AT_KEYS, t_hi = p_last / AT_KEYS;
    const int per_part = (t_hi - t_all + nsplit) / nsplit;        // ceil(tiles / nsplit)
    const int t_lo = t_all + part * per_part;                      // this block's first tile
    if (t_lo > t_hi) return;                                    // a part without tiles
    const int n_tiles = min(t_hi, t_lo + per_part - 1) - t_lo + 1;
    const int page_shift = 31 - __clz(page_size);
    const int ppt = AT_KEYS >> page_shift;                      // pages per tile (1..16)
    const unsigned page_bytes = (unsigned)page_size * HD * 2u;

    constexpr int TILE = AT_KEYS * HD;                          // elements of a K or V tile
    extern __shared__ __align__(16) unsigned char smem_raw[];   // aligned by hand
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    bf16* q_tile = (bf16*)base;                                 // [128 rows][64]
    bf16* kv_ring = q_tile + AT_ROWS * HD;                      // [stages][K tile, V tile]
    bf16* p_tile = kv_ring + (size_t)AT_STAGES * 2 * TILE;      // [128 rows][64 keys]
    __shared__ __align__(8) unsigned long long q_bar, s_bar, pv_bar, s_read, p_ready;
    __shared__ __align__(8) unsigned long long k_full[AT_STAGES], k_empty[AT_STAGES];
    __shared__ __align__(8) unsigned long long v_full[AT_STAGES], v_empty[AT_STAGES];
    __shared__ unsigned tmem_base_smem;
    __shared__ volatile int failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        failed = 0;
        at_mbar_init(&q_bar, 1);
        at_mbar_init(&s_bar, 1);
        at_mbar_init(&pv_bar, 1);
        at_mbar_init(&s_read, AT_ROWS);
        at_mbar_init(&p_ready, AT_ROWS);
        for (int s = 0; s < AT_STAGES; ++s) {
            at_mbar_init(&k_full[s], 1);
            at_mbar_init(&k_empty[s], 1);
            at_mbar_init(&v_full[s], 1);
            at_mbar_init(&v_empty[s], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(at_smem(&tmem_base_smem)), "r"(128u));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = tmem_base_smem;
    const unsigned tmem_s = tmem_base, tmem_o = tmem_base + AT_KEYS;

    if (warp == 4) {
        // ---- producer warp: Q once, then keys and values, each as soon as its stage is free.
        // A key stage is free when its S = Q K^T is done, a value stage when its P V is done,
        // so the keys run ahead of the values.  The warp polls both "stage free" barriers
        // without blocking on either (a blocked wait for values would hold back the keys).
        if (lane == 0) {
            at_mbar_expect_tx(&q_bar, (unsigned)(q_block * G * HD * 2));
            at_tma_3d(q_tile, &map_q, 0, g * G, qs + q0, &q_bar);
        }
        int next_k = 0, next_v = 0;
        const long long t_start = clock64();
        long long t_progress = t_start;
        auto copy_tile = [&](int n, bool values) {
            const int s = n % AT_STAGES;
            unsigned long long* full = values ? &v_full[s] : &k_full[s];
            bf16* dst = kv_ring + (size_t)s * 2 * TILE + (values ? TILE : 0);
            const int blk = (t_lo + n) * ppt + lane;
            int page = -1;
            if (lane < ppt && blk < max_blocks && (blk << page_shift) < clen)
                page = block_table[(size_t)r * max_blocks + blk];
            const unsigned have = __ballot_sync(0xffffffffu, lane < ppt && page >= 0);
            const unsigned miss = __ballot_sync(0xffffffffu, lane < ppt && page < 0);
            if (miss) {                     // pages past the context or given back: zeros
                const uint4 z = make_uint4(0, 0, 0, 0);
                for (int pi = 0; pi < ppt; ++pi) {
                    if (!((miss >> pi) & 1u)) continue;
                    uint4* dz = (uint4*)(dst + (size_t)pi * page_size * HD);
                    for (int i = lane; i < (int)(page_bytes / 16); i += 32) dz[i] = z;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            __syncwarp();
            if (lane == 0) at_mbar_expect_tx(full, (unsigned)__popc(have) * page_bytes);
            __syncwarp();
            if (lane < ppt && page >= 0)
                at_tma_3d(dst + (size_t)lane * page_size * HD, values ? &map_v : &map_k, 0, g,
                          page << page_shift, full);
        };
        while ((next_k < n_tiles || next_v < n_tiles) && !failed) {
            bool did = false;
            if (next_k < n_tiles) {
                bool free_k = next_k < AT_STAGES;
                if (!free_k && lane == 0)
                    free_k = at_mbar_try_wait(&k_empty[next_k % AT_STAGES],
                                              (unsigned)((next_k / AT_STAGES) - 1) & 1u);
                if (__shfl_sync(0xffffffffu, (int)free_k, 0)) {
                    copy_tile(next_k++, false);
                    did = true;
                }
            }
            if (next_v < n_tiles) {
                bool free_v = next_v < AT_STAGES;
                if (!free_v && lane == 0)
                    free_v = at_mbar_try_wait(&v_empty[next_v % AT_STAGES],
                                              (unsigned)((next_v / AT_STAGES) - 1) & 1u);
                if (__shfl_sync(0xffffffffu, (int)free_v, 0)) {
                    copy_tile(next_v++, true);
                    did = true;
                }
            }
            const long long now = clock64();
            if (did) {
                t_progress = now;
            } else if (now - t_progress > AT_WAIT_CYCLES) {      // bounded: nothing freed for 0.2 s
                if (lane == 0 && !failed) { failed = 1; atomicCAS(status, 0, 21); }
                __syncwarp();
                break;
            }
        }
        if (failed && lane == 0) {
            // no copy may arrive after the block has left: wait (bounded) for the armed stages
            const long long t0 = clock64();
            for (int n = max(0, next_k - AT_STAGES); n < next_k; ++n) {
                bool ok = false;
                while (!ok && clock64() - t0 < AT_WAIT_CYCLES)
                    ok = at_mbar_try_wait(&k_full[n % AT_STAGES], (unsigned)(n / AT_STAGES) & 1u);
            }
            for (int n = max(0, next_v - AT_STAGES); n < next_v; ++n) {
                bool ok = false;
                while (!ok && clock64() - t0 < AT_WAIT_CYCLES)
                    ok = at_mbar_try_wait(&v_full[n % AT_STAGES], (unsigned)(n / AT_STAGES) & 1u);
            }
            bool ok = false;
            while (!ok && clock64() - t0 < AT_WAIT_CYCLES) ok = at_mbar_try_wait(&q_bar, 0);
        }
    } else if (warp == 5) {
        // ---- MMA issuer (thread 0 of the sixth warp) ----------------------------------------
        // S = Q K^T of tile n + 1 is issued as soon as every row has read S of tile n out of
        // TMEM, so it runs while the rows do their softmax; O += P V of tile n when its P is
        // written.  instruction descriptors: D float32, A and B bfloat16; N >> 3 at bit 17,
        // M >> 4 at bit 24; bit 16: B is MN-major (V lies [key][dim]).
        if (lane == 0) {
            const unsigned idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) |
                                      ((unsigned)(AT_KEYS >> 3) << 17) | ((unsigned)(AT_ROWS >> 4) << 24);
            const unsigned idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                                      ((unsigned)(HD >> 3) << 17) | ((unsigned)(AT_ROWS >> 4) << 24);
            auto give_up = [&]() {
                if (!failed) { failed = 1; atomicCAS(status, 0, 21); }
            };
            auto issue_qk = [&](int n) {
                const int s = n % AT_STAGES;
                if (!failed && !at_mbar_wait(&k_full[s], (unsigned)(n / AT_STAGES) & 1u, &failed)) give_up();
                if (!failed) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned long long a0 = at_desc(q_tile);
                    const unsigned long long b0 = at_desc(kv_ring + (size_t)s * 2 * TILE);
#pragma unroll
                    for (int k = 0; k < HD / 16; ++k)              // 32 bytes per K = 16 step
                        at_mma(tmem_s, a0 + 2 * k, b0 + 2 * k, idesc_qk, k != 0);
                }
                at_commit(&k_empty[s]);                             // the key stage is free again
                at_commit(&s_bar);
            };
            if (!at_mbar_wait(&q_bar, 0, &failed)) give_up();
            issue_qk(0);
            for (int n = 0; n < n_tiles; ++n) {
                const int s = n % AT_STAGES;
                if (n + 1 < n_tiles) {
                    if (!failed && !at_mbar_wait(&s_read, (unsigned)n & 1u, &failed)) give_up();
                    issue_qk(n + 1);
                }
                if (!failed && !at_mbar_wait(&p_ready, (unsigned)n & 1u, &failed)) give_up();
                if (!failed && !at_mbar_wait(&v_full[s], (unsigned)(n / AT_STAGES) & 1u, &failed)) give_up();
                if (!failed) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned long long a0 = at_desc(p_tile);
                    const unsigned long long b0 = at_desc(kv_ring + (size_t)s * 2 * TILE + TILE);
#pragma unroll
                    for (int k = 0; k < AT_KEYS / 16; ++k)
                        // P: 32 bytes per K = 16 step; V: 16 keys = 16 rows of 128 bytes per step
                        at_mma(tmem_o, a0 + 2ull * k, b0 + (unsigned long long)(k * (16 * 128 >> 4)),
                               idesc_pv, (n | k) != 0);
                }
                at_commit(&v_empty[s]);                             // the value stage is free again
                at_commit(&pv_bar);
            }
        }
    } else {
        // ---- rows: thread `tid` owns row tid = token * G + head ---------------------------
        // The four warps never meet at a block barrier inside the loop: they wait for S
        // (`s_bar`) and for the previous P V (`pv_bar`), and tell the issuer by mbarrier
        // arrivals that S is read (`s_read`) and P written (`p_ready`).  A wait that runs out
        // sets `failed`; every later wait then returns at once, the threads still walk every
        // tile and arrive everywhere, and the output is not written.
        const int m = tid;
        const int tok = m / G, head = m - tok * G;
        const bool row_ok = tok < n_tok;
        const int p_row = row_ok ? p_first + tok : -1;          // its own position: the last key
        const int lo_row = window > 0 ? max(0, p_row - window + 1) : 0;
        const unsigned lane_base = ((unsigned)(warp * 32)) << 16;
        float m_run = -INFINITY, l_run = 0.f;                   // exponent offset (scaled) and sum
        for (int n = 0; n < n_tiles; ++n) {
            if (!at_mbar_wait(&s_bar, (unsigned)n & 1u, &failed) && !failed) {
                failed = 1;
                atomicCAS(status, 0, 21);
            }
            __syncwarp();
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float sv[AT_KEYS];
            at_tmem_ld64(tmem_s + lane_base, sv);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            at_mbar_arrive(&s_read);                                // S may be overwritten
            // masked where this tile can hold keys the row may not see (a tile wholly inside
            // every row's range needs no compare)
            const int key0 = (t_lo + n) * AT_KEYS;
            if (key0 + AT_KEYS - 1 > p_first || (window > 0 && key0 < p_last - window + 1)) {
#pragma unroll
                for (int j = 0; j < AT_KEYS; ++j) {
                    const int key = key0 + j;
                    if (key > p_row || key < lo_row) sv[j] = -INFINITY;
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains, not one
#pragma unroll
            for (int j = 0; j < AT_KEYS; j += 4) {
                mx4[0] = fmaxf(mx4[0], sv[j]);
                mx4[1] = fmaxf(mx4[1], sv[j + 1]);
                mx4[2] = fmaxf(mx4[2], sv[j + 2]);
                mx4[3] = fmaxf(mx4[3], sv[j + 3]);
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
            // The exponent's offset follows the row maximum lazily: it moves only when the
            // maximum has grown by more than 2^8 since it was set (P then stays below 256,
            // exact in bfloat16 and harmless in the float32 sums), so O is rescaled on few
            // tiles; the final O / l does not depend on the offsets chosen on the way.
            const bool moved = mx > m_run + 8.f || (m_run == -INFINITY && mx > -INFINITY);
            const float m_new = moved ? mx : m_run;
            const float off = m_new == -INFINITY ? 0.f : m_new;
            const float corr = moved ? at_exp2(m_run - off) : 1.f;  // m_run = -inf -> 0
            m_run = m_new;
            // P = 2^(S * scale - offset) as bfloat16, kept in registers while the previous
            // tile's P V may still be running
            unsigned pk[AT_KEYS / 2];
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < AT_KEYS; j += 2) {
                const float e0 = at_exp2(fmaf(sv[j], scale_log2, -off));
                const float e1 = at_exp2(fmaf(sv[j + 1], scale_log2, -off));
                sum4[(j >> 1) & 3] += e0 + e1;
                const __nv_bfloat162 pr = __floats2bfloat162_rn(e0, e1);
                pk[j >> 1] = *(const unsigned*)&pr;
            }
            l_run = l_run * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            // the previous tile's P V must be done before O is touched and P overwritten
            if (n > 0 && !at_mbar_wait(&pv_bar, (unsigned)(n - 1) & 1u, &failed) && !failed) {
                failed = 1;
                atomicCAS(status, 0, 21);
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (n > 0 && __any_sync(0xffffffffu, moved)) {          // O *= corr, row by row
#pragma unroll
                for (int c = 0; c < HD; c += 16) {
                    float v[16];
                    at_tmem_ld16(tmem_o + lane_base + (unsigned)c, v);
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] *= corr;
                    at_tmem_st16(tmem_o + lane_base + (unsigned)c, v);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            {
                // row m of the P tile: 128 bytes whose 16-byte chunks are XOR-swizzled with m & 7
                unsigned char* row = (unsigned char*)p_tile + (size_t)m * 128;
#pragma unroll
                for (int ch = 0; ch < 8; ++ch)
                    *(uint4*)(row + ((ch ^ (m & 7)) << 4)) =
                        make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            at_mbar_arrive(&p_ready);
        }
        const bool done = at_mbar_wait(&pv_bar, (unsigned)(n_tiles - 1) & 1u, &failed);
        if (__all_sync(0xffffffffu, done && !failed)) {         // one answer per warp: the reads
                                                                // below are warp-wide
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (nsplit > 1) {
                // this part's rows as they stand: O unnormalised, the offset and the sum
                const size_t slot = (((size_t)r_local * gridDim.y + blockIdx.y) * gridDim.x + g) * nsplit + part;
                float* po = part_o + (slot * AT_ROWS + m) * HD;
                if (row_ok) part_ml[slot * AT_ROWS + m] = make_float2(m_run, l_run);
#pragma unroll
                for (int c = 0; c < HD; c += 16) {
                    float v[16];
                    at_tmem_ld16(tmem_o + lane_base + (unsigned)c, v);
                    if (row_ok) {
#pragma unroll
                        for (int j = 0; j < 16; j += 4)
                            *(float4*)(po + c + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    }
                }
            } else {
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            bf16* dst = out + (size_t)(qs + q0 + tok) * num_heads * HD + (size_t)(g * G + head) * HD;
#pragma unroll
            for (int c = 0; c < HD; c += 16) {
                float v[16];
                at_tmem_ld16(tmem_o + lane_base + (unsigned)c, v);
                if (row_ok) {
                    unsigned pk[8];
#pragma unroll
                    for (int j = 0; j < 16; j += 2) {
                        const __nv_bfloat162 pr = __floats2bfloat162_rn(v[j] * inv, v[j + 1] * inv);
                        pk[j >> 1] = *(const unsigned*)&pr;
                    }
                    *(uint4*)(dst + c) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    *(uint4*)(dst + c + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                }
            }
            }
        } else if (!failed) {
            failed = 1;
            atomicCAS(status, 0, 21);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(128u));
    }
}

// The parts of a block of query tokens put together, in order.  A thread owns four columns of
// one row and requests every part's values before it uses any (one memory latency, however
// many parts); 16 rows a block, so blockIdx.z = request * 8 + sixteen rows of the 128.  The
// same arithmetic as the kernel above, so a part that had no tiles is skipped here too.
#define AT_MAX_PARTS 16
template <int HD>
__global__ void __launch_bounds__(16 * (HD / 4)) paged_attention_prefill_merge_kernel(
    const float* __restrict__ part_o, const float2* __restrict__ part_ml,
    const int* __restrict__ q_start, const int* __restrict__ ctx_lens, bf16* __restrict__ out,
    int first_req, int num_heads, int num_kv_heads, int q_block, int window, int nsplit) {
    rv_pdl_prologue();
    constexpr int CH = HD / 4;                                  // 4-column chunks of a row
    const int r_local = (int)blockIdx.z / (AT_ROWS / 16), rows0 = ((int)blockIdx.z % (AT_ROWS / 16)) * 16;
    const int r = first_req + r_local, g = blockIdx.x;
    const int clen = ctx_lens[r];
    const int qs = q_start[r];
    const int qlen = q_start[r + 1] - qs;
    const int nqb = (qlen + q_block - 1) / q_block;
    if ((int)blockIdx.y >= nqb || clen == 0) return;
    const int qb = nqb - 1 - blockIdx.y;
    const int G = num_heads / num_kv_heads;
    const int q0 = qb * q_block;
    const int n_tok = min(q_block, qlen - q0);
    const int p_first = clen - qlen + q0, p_last = p_first + n_tok - 1;
    const int key_lo = window > 0 ? max(0, p_first - window + 1) : 0;
    const int t_all = key_lo / AT_KEYS, t_hi = p_last / AT_KEYS;
    const int per_part = (t_hi - t_all + nsplit) / nsplit;
    const int m = rows0 + (int)threadIdx.x / CH, c = ((int)threadIdx.x % CH) * 4;
    const int tok = m / G, head = m - tok * G;
    if (tok >= n_tok) return;
    const size_t slot0 = (((size_t)r_local * gridDim.y + blockIdx.y) * gridDim.x + g) * nsplit;
    float2 ml[AT_MAX_PARTS];
    float4 v[AT_MAX_PARTS];
#pragma unroll
    for (int p = 0; p < AT_MAX_PARTS; ++p) {
        const bool there = p < nsplit && t_all + p * per_part <= t_hi;
        ml[p] = there ? part_ml[(slot0 + p) * AT_ROWS + m] : make_float2(-INFINITY, 0.f);
        v[p] = there ? *(const float4*)(part_o + ((slot0 + p) * AT_ROWS + m) * HD + c)
                     : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float M = -INFINITY;
#pragma unroll
    for (int p = 0; p < AT_MAX_PARTS; ++p)
        if (ml[p].y > 0.f) M = fmaxf(M, ml[p].x);
    float L = 0.f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int p = 0; p < AT_MAX_PARTS; ++p) {
        if (ml[p].y > 0.f) {                                    // something visible in this part
            const float w = at_exp2(ml[p].x - M);
            L += ml[p].y * w;
            o.x += v[p].x * w; o.y += v[p].y * w; o.z += v[p].z * w; o.w += v[p].w * w;
        }
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    bf16* dst = out + (size_t)(qs + q0 + tok) * num_heads * HD + (size_t)(g * G + head) * HD + c;
    const __nv_bfloat162 lo = __floats2bfloat162_rn(o.x * inv, o.y * inv);
    const __nv_bfloat162 hi = __floats2bfloat162_rn(o.z * inv, o.w * inv);
    *(uint2*)dst = make_uint2(*(const unsigned*)&lo, *(const unsigned*)&hi);
}

// ---- host side ----------------------------------------------------------------------------
static thread_local char g_at_error[512] = "";
static int at_fail(const char* msg) {
    snprintf(g_at_error, sizeof(g_at_error), "%s", msg);
    return 1;
}
#define AT_CAT2(a, b) a##b
#define AT_CAT(a, b) AT_CAT2(a, b)
#define AT_SYM(name) AT_CAT(AT_CAT(name, _hd), RV_HD)

extern "C" const char* AT_SYM(rv_attention_tcgen05_last_error)() { return g_at_error; }

typedef CUresult (*AtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                               const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                               const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// [rows][mid][64] bfloat16 with `mid_stride_bytes` between rows: box [box_rows, box_mid, 64].
static int at_map(CUtensorMap* map, const void* ptr, long long rows, int mid, long long row_bytes,
                  int box_rows, int box_mid) {
    static AtEncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) !=
                cudaSuccess || qr != cudaDriverEntryPointSuccess)
            return at_fail("paged_attention_prefill_tcgen05: cuTensorMapEncodeTiled is not available");
        fn = (AtEncodeFn)p;
    }
    cuuint64_t dims[3] = {RV_HD, (cuuint64_t)mid, (cuuint64_t)rows};
    cuuint64_t strides[2] = {RV_HD * 2, (cuuint64_t)row_bytes};
    cuuint32_t box[3] = {RV_HD, (cuuint32_t)box_mid, (cuuint32_t)box_rows};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides,
                    box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return at_fail("paged_attention_prefill_tcgen05: cuTensorMapEncodeTiled failed");
    return 0;
}

// A launch with fewer blocks than two an SM shares the key tiles of every block of query tokens
// out over several blocks, so that a short portion at the end of a long context is not one long
// chain of tiles on a few SMs (256 tokens at the end of 4,096: 64.7 -> 31.7 us; 512 at the end of
// 2,048: 35.6 -> 31.6); the parts are put together by the merge kernel.  About two blocks an SM
// in all (with three the blocks slow one another down as much as the sharing out gains: 1,024
// tokens at the end of 4,096 78.7 -> 85.1 us), at most 16 parts: the scratch for the parts is bounded by the size below.
#define AT_PART_BYTES ((size_t)AT_ROWS * (RV_HD * 4 + 8))
extern "C" long long AT_SYM(rv_paged_attention_prefill_tcgen05_scratch_bytes)(int n_sms) {
    return (long long)(6 * (size_t)(n_sms > 0 ? n_sms : 1) * AT_PART_BYTES);
}

static int at_parts(long long blocks, int max_ctx_len, int max_q_len, int n_sms, long long scratch_bytes) {
    static const int forced = [] {
        const char* e = getenv("RVLLM_PREFILL_SPLIT");
        return e && *e ? atoi(e) : 0;
    }();
    const long long places = 2ll * n_sms;
    int parts = forced > 0 ? forced : (int)((places + blocks / 2) / blocks);
    // the tiles every block of query tokens has before its own: a whole prompt (none before it)
    // is a triangle of mostly short blocks, which sharing out only burdens (1,000 tokens alone:
    // 22.7 -> 29.2 us with two parts); four such tiles to a part at least
    const int before = (max_ctx_len > max_q_len ? max_ctx_len - max_q_len : 0) / AT_KEYS;
    if (forced <= 0 && parts > before / 4) parts = before / 4;
    if (parts > AT_MAX_PARTS) parts = AT_MAX_PARTS;
    while (parts > 1 && (blocks * parts > 3 * places ||
                         (long long)(blocks * parts * AT_PART_BYTES) > scratch_bytes))
        --parts;
    return parts < 1 ? 1 : parts;
}

// Requests [first_req, first_req + n_reqs), the longest bringing max_q_len tokens and holding
// max_ctx_len; `q` is the q|k|v buffer [n_tokens, q_stride] (the query heads first), `out` is
// [n_tokens, heads * 64]; `scratch` (may be null: no sharing out) holds the parts.
extern "C" int AT_SYM(rv_paged_attention_prefill_tcgen05)(
    const void* q, int q_stride, int n_tokens, const void* k_cache, const void* v_cache,
    long long total_slots, const int* block_table, int max_blocks, const int* q_start,
    const int* ctx_lens, void* out, int first_req, int n_reqs, int max_q_len, int max_ctx_len,
    int num_heads, int num_kv_heads, int page_size, float scale, int window, int* status,
    void* scratch, long long scratch_bytes, int n_sms, void* stream) {
    if (n_reqs == 0 || max_q_len == 0) return 0;
    if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads || n_reqs < 0)
        return at_fail("paged_attention_prefill_tcgen05: bad head counts");
    const int G = num_heads / num_kv_heads;
    if (G > AT_ROWS) return at_fail("paged_attention_prefill_tcgen05: more than 128 heads per group");
    if (page_size < 8 || page_size > AT_KEYS || (page_size & (page_size - 1)))
        return at_fail("paged_attention_prefill_tcgen05: pages of 8, 16, 32 or 64 tokens only");
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) % 16 ||
        q_stride % RV_HD)
        return at_fail("paged_attention_prefill_tcgen05: buffers must be 16-byte aligned and rows whole heads");
    const int q_block = AT_ROWS / G;                             // query tokens per block
    CUtensorMap map_q, map_k, map_v;
    if (at_map(&map_q, q, n_tokens, q_stride / RV_HD, (long long)q_stride * 2, q_block, G)) return 1;
    if (at_map(&map_k, k_cache, total_slots, num_kv_heads, (long long)num_kv_heads * RV_HD * 2,
               page_size, 1))
        return 1;
    if (at_map(&map_v, v_cache, total_slots, num_kv_heads, (long long)num_kv_heads * RV_HD * 2,
               page_size, 1))
        return 1;
    const size_t smem = (size_t)(AT_ROWS * RV_HD + AT_STAGES * 2 * AT_KEYS * RV_HD + AT_ROWS * AT_KEYS) *
                            sizeof(bf16) + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(paged_attention_prefill_tcgen05_kernel<RV_HD>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return at_fail(cudaGetErrorString(e));
        configured = true;
    }
    const int nqb = (max_q_len + q_block - 1) / q_block;
    const long long blocks = (long long)num_kv_heads * nqb * n_reqs;
    const int parts = scratch && n_sms > 0 ? at_parts(blocks, max_ctx_len, max_q_len, n_sms, scratch_bytes) : 1;
    if ((long long)n_reqs * (parts > AT_ROWS / 16 ? parts : AT_ROWS / 16) > 65535)
        return at_fail("paged_attention_prefill_tcgen05: too many requests");
    float* part_o = (float*)scratch;
    float2* part_ml = (float2*)((char*)scratch + (size_t)blocks * parts * AT_ROWS * RV_HD * 4);
    rv_launch(paged_attention_prefill_tcgen05_kernel<RV_HD>, dim3(num_kv_heads, nqb, n_reqs * parts),
              dim3(192), smem, (cudaStream_t)stream, map_q, map_k, map_v, block_table, max_blocks,
              q_start, ctx_lens, (bf16*)out, first_req, num_heads, num_kv_heads, q_block, page_size,
              scale * 1.4426950408889634f, window, status, parts, part_o, part_ml);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return at_fail(cudaGetErrorString(e));
    if (parts > 1) {
        rv_launch(paged_attention_prefill_merge_kernel<RV_HD>,
                  dim3(num_kv_heads, nqb, n_reqs * (AT_ROWS / 16)), dim3(16 * (RV_HD / 4)), 0,
                  (cudaStream_t)stream, (const float*)part_o, (const float2*)part_ml,
                  q_start, ctx_lens, (bf16*)out, first_req, num_heads, num_kv_heads, q_block, window, parts);
        e = cudaGetLastError();
        if (e != cudaSuccess) return at_fail(cudaGetErrorString(e));
    }
    return 0;
}
