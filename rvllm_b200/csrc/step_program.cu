// A decode step as one resident kernel: a list of operations ("step program") that every SM
// walks together, so that weights stream from HBM without a pause between the products.
//
// Why.  A decode step of a few tokens is bound by reading every weight once.  Run as one launch
// per operation, each product pays for the gap between kernels: its blocks start, fill their
// copy rings, stream, reduce, leave, and the small kernels between two products move kilobytes
// while no weight is in flight.  Here one block per SM stays resident for a whole stretch of
// the step.  In each block a producer thread walks the list *ahead* of the computation and
// keeps a ring of weight tiles full (TMA, cp.async.bulk.tensor.2d), bounded only by the ring's
// size: while the blocks meet at the barrier between two operations, or run a small
// elementwise operation, the next products' weights are already on their way.
//
// The operations.  A product y = x . W^T (few tokens; bfloat16 operands, float32 sums) is cut
// into items (128 rows of W) x (a slice of K of at most 16 blocks of 64); an item is
// tcgen05.mma instructions (M = 128 weight rows, N = 16 token columns, accumulator in TMEM)
// over the ring's tiles and the item's slice of x in shared memory; the float32 tile goes to a
// partial-sum buffer [slice][token][row] in global memory.  Every product is followed by an
// elementwise operation that adds the slices in a fixed order while it loads them, so the sum
// is deterministic and no atomics are used:
//   RESID   stream += sum (or stream = embedding rows); emits the stream times the next norm's
//           weight in bfloat16, and per-token sums of squares by column slice.  The norm's
//           division is left to whoever consumes the product of those rows: a per-token
//           factor commutes with the product.
//   CONV    the gated short convolution for one token per request, with its state update
//   QK      per-head q/k norm, rotation, query rows out, keys and values into their pages
//   SWIGLU  silu(gate) * up
//   LOGITS  the head's product times the final norm's factor, float32
// Attention itself is not in the list: the host runs a stretch up to the QK operation, then
// the decode attention kernels, then the next stretch.
//
// Meeting between operations.  Operation k may read what operation k-1 wrote once every block
// has finished k-1.  Each block's worker threads add one to `counters[k]` (after a fence) when
// their share of k is done, and whoever needs k's results polls until the count equals the
// grid size.  The launch is cooperative, so all blocks are resident and the wait ends; it is
// bounded all the same (RV_WAIT_CYCLES), and a block that gives up records a code in `status`,
// stops all its roles, waits for its copies in flight, frees its TMEM and returns, and every
// other block does the same as soon as it sees the status.  The last block to arrive at k
// clears counters[k-1], which nobody polls any more, so the counters are zero again when the
// kernel ends.
//
// Roles in a block (192 threads): warp 0 lane 0 copies weight tiles; warp 1 lane 0 waits for
// the inputs of a product, copies the item's slice of x (TMA) and issues the MMAs; warps 2-5
// read accumulators from TMEM (two of them, so an item's sums are written while the next
// item's MMAs run) and carry out the elementwise operations.
//
// Reference counterpart: the sequence of cuBLAS calls and small kernels of one forward pass
// (src/cuda/model.rs:560-790).  Plain reference: tests/plain_ops.py, operation by operation.
#include <new>
#include <vector>

#include "tcgen05_common.cuh"

#define SP_BM 128
#define SP_BK 64
#define SP_NPAD 16                    // token columns of an MMA
#define SP_MAX_KB 16                  // K blocks of an item's slice: 32 KB of x
#define SP_W_BYTES (SP_BM * SP_BK * 2)
#define SP_X_BYTES (SP_NPAD * SP_BK * 2)
#define SP_ACT_BYTES (SP_MAX_KB * SP_X_BYTES)
#define SP_MAX_STAGES 12
#define SP_THREADS 192
#define SP_WORKERS 128
#define SP_MAX_TAPS 8
#define SP_SLICE 64                   // columns per sum-of-squares slice

enum { SP_GEMM = 1, SP_RESID = 2, SP_CONV = 3, SP_QK = 4, SP_SWIGLU = 5, SP_LOGITS = 6 };

struct __align__(64) RvStepOp {
    CUtensorMap map_w;            // GEMM: W [N, K]
    CUtensorMap map_x;            // GEMM: x [16, K]
    int type;
    int M;                        // live tokens (<= 16)
    int N, K;                     // GEMM: rows of W, width; elementwise: N = width of the partial rows
    int tiles, splits, kblocks;   // GEMM
    int part_splits;              // slices to add when reading `part`
    float* part;                  // GEMM: written [splits][16][N]; elementwise: read
    // per-token factor 1 / sqrt(sum over slices of ss_in / dim + eps); n_slices 0: none
    const float* ss_in;
    int n_slices;
    float eps, dim;
    // RESID
    float* resid;                 // [16][N] float32
    bf16* xw;                     // [16][N] stream * w_next
    float* ss_out;                // [slices][16]
    const float* w_next;          // [N]
    const bf16* embed;            // non-null: stream = embed[token_ids[t]] * embed_scale
    const int* token_ids;
    const float* bias;            // [N] added with the sum, or null
    float embed_scale;
    int vocab;
    // CONV (N = 3 * hidden)
    const float* filter;          // [hidden][taps]
    const float* in_bias;         // [3 hidden] or null
    const float* conv_bias;       // [hidden] or null
    float* state;                 // [slots][taps - 1][hidden]
    const int* state_slot;        // [tokens], -1: none
    const int* start_pos;         // [tokens]
    int taps, hidden;
    // output rows of CONV / SWIGLU (bfloat16 [16][width]) and QK (query rows [16][N])
    bf16* act_out;
    // QK (N = (heads + 2 kv heads) * head_dim)
    const float* q_weight;
    const float* k_weight;
    const float* cos_table;
    const float* sin_table;
    const int* positions;
    const int* slot_mapping;
    bf16* k_cache;
    bf16* v_cache;
    float qk_eps;
    int num_heads, num_kv_heads, head_dim;
    // LOGITS
    float* logits;                // [16][N]
};

// ---- small device helpers -------------------------------------------------------------------
__device__ __forceinline__ void sp_fence_proxy_async() {
    asm volatile("fence.proxy.async;" ::: "memory");
}
__device__ __forceinline__ unsigned sp_ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long sp_globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void sp_worker_sync() {
    asm volatile("bar.sync 1, %0;" ::"n"(SP_WORKERS) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

struct SpShared {
    unsigned long long full_bar[SP_MAX_STAGES];
    unsigned long long empty_bar[SP_MAX_STAGES];
    unsigned long long act_full, act_free;
    unsigned long long accum_full[2], accum_empty[2];
    unsigned tmem_base;
    volatile int failed;
    volatile int stop;            // `failed` as the workers sampled it together
    float rs[SP_NPAD];
};

__device__ __forceinline__ void sp_fail(SpShared* sh, int* status, int code) {
    if (!sh->failed) {
        sh->failed = 1;
        atomicCAS(status, 0, code);
    }
}

// Wait until every block has finished operation `k` (counters[k] == grid size).
__device__ bool sp_wait_done(const unsigned* counter, unsigned target, SpShared* sh, int* status) {
    if (sp_ld_acquire(counter) >= target) return true;
    const long long start = clock64();
    for (unsigned i = 1;; ++i) {
        if (sp_ld_acquire(counter) >= target) return true;
        if (sh->failed) return false;
        if ((i & 31u) == 0) {
            if (*(volatile int*)status != 0) {       // another block gave up
                sh->failed = 1;
                return false;
            }
            if (clock64() - start > RV_WAIT_CYCLES) return false;
        }
    }
}

// The items of a product that block `cta` of `G` takes: one K slice, tiles first, first + stride...
__device__ __forceinline__ bool sp_items(const RvStepOp* op, int cta, int G, int& split, int& first,
                                         int& stride, int& kb0, int& kb1) {
    const int S = op->splits;
    stride = G / S;
    if (cta >= stride * S) return false;
    split = cta % S;
    first = cta / S;
    kb0 = (int)((long long)op->kblocks * split / S);
    kb1 = (int)((long long)op->kblocks * (split + 1) / S);
    return first < op->tiles && kb1 > kb0;
}

// 1 / sqrt(mean square + eps) of every token's normalised input, into shared memory.
__device__ __forceinline__ void sp_row_scales(const RvStepOp* op, SpShared* sh, int wtid) {
    if (wtid < SP_NPAD) {
        float r = 1.f;
        if (op->n_slices > 0) {
            float ss = 0.f;
            for (int s = 0; s < op->n_slices; ++s) ss += op->ss_in[s * SP_NPAD + wtid];
            r = 1.f / sqrtf(ss / op->dim + op->eps);
        }
        sh->rs[wtid] = r;
    }
    sp_worker_sync();
}

__device__ __forceinline__ float sp_sum_parts(const float* part, int splits, size_t stride, size_t at) {
    float v = 0.f;
    for (int s = 0; s < splits; ++s) v += part[s * stride + at];
    return v;
}

// ---- elementwise operations ---------------------------------------------------------------
__device__ void sp_resid(const RvStepOp* op, int cta, int wtid) {
    const int H = op->N;
    const int slices = (H + SP_SLICE - 1) / SP_SLICE;
    if (cta >= slices) return;
    const int t = wtid >> 3, c0 = cta * SP_SLICE + (wtid & 7) * 8;
    const bool live = t < op->M && c0 < H;           // H is a multiple of 8
    float ss = 0.f;
    if (live) {
        float v[8];
        float* r = op->resid + (size_t)t * H + c0;
        if (op->embed) {
            int row = op->token_ids[t];
            row = row < 0 ? 0 : (row >= op->vocab ? op->vocab - 1 : row);
            const uint4 raw = *(const uint4*)(op->embed + (size_t)row * H + c0);
            const __nv_bfloat162* h2 = (const __nv_bfloat162*)&raw;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(h2[i]);
                v[2 * i] = f.x * op->embed_scale;
                v[2 * i + 1] = f.y * op->embed_scale;
            }
        } else {
            const float4 a = *(const float4*)r, b = *(const float4*)(r + 4);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
            v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
            const size_t stride = (size_t)SP_NPAD * H;
            for (int s = 0; s < op->part_splits; ++s) {
                const float* p = op->part + s * stride + (size_t)t * H + c0;
                const float4 pa = *(const float4*)p, pb = *(const float4*)(p + 4);
                v[0] += pa.x; v[1] += pa.y; v[2] += pa.z; v[3] += pa.w;
                v[4] += pb.x; v[5] += pb.y; v[6] += pb.z; v[7] += pb.w;
            }
            if (op->bias) {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] += op->bias[c0 + i];
            }
        }
        *(float4*)r = make_float4(v[0], v[1], v[2], v[3]);
        *(float4*)(r + 4) = make_float4(v[4], v[5], v[6], v[7]);
        uint4 out;
        __nv_bfloat162* o2 = (__nv_bfloat162*)&out;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            o2[i] = __floats2bfloat162_rn(v[2 * i] * op->w_next[c0 + 2 * i],
                                          v[2 * i + 1] * op->w_next[c0 + 2 * i + 1]);
            ss += v[2 * i] * v[2 * i] + v[2 * i + 1] * v[2 * i + 1];
        }
        *(uint4*)(op->xw + (size_t)t * H + c0) = out;
    }
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    ss += __shfl_xor_sync(0xffffffffu, ss, 4);
    if ((wtid & 7) == 0) op->ss_out[cta * SP_NPAD + t] = ss;
}

__device__ void sp_conv(const RvStepOp* op, SpShared* sh, int cta, int G, int wtid) {
    sp_row_scales(op, sh, wtid);
    const int H = op->hidden, taps = op->taps, hist = taps - 1;
    const size_t pstride = (size_t)SP_NPAD * op->N;
    for (int e = cta * SP_WORKERS + wtid; e < op->M * H; e += G * SP_WORKERS) {
        const int t = e / H, c = e - t * H;
        const float rs = sh->rs[t];
        const size_t row = (size_t)t * op->N;
        float b = rs * sp_sum_parts(op->part, op->part_splits, pstride, row + c);
        float g = rs * sp_sum_parts(op->part, op->part_splits, pstride, row + H + c);
        float x = rs * sp_sum_parts(op->part, op->part_splits, pstride, row + 2 * H + c);
        if (op->in_bias) {
            b += op->in_bias[c];
            g += op->in_bias[H + c];
            x += op->in_bias[2 * H + c];
        }
        const float bx = b * x;
        const int slot = op->state && hist > 0 ? op->state_slot[t] : -1;
        const bool has = slot >= 0 && op->start_pos[t] > 0;
        float* st = slot >= 0 ? op->state + (size_t)slot * hist * H + c : nullptr;
        float win[SP_MAX_TAPS - 1];
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < SP_MAX_TAPS - 1; ++k) {
            win[k] = (k < hist && has) ? st[(size_t)k * H] : 0.f;
            if (k < hist) acc += op->filter[(size_t)c * taps + k] * win[k];
        }
        acc += op->filter[(size_t)c * taps + hist] * bx;
        if (op->conv_bias) acc += op->conv_bias[c];
        op->act_out[(size_t)t * H + c] = __float2bfloat16_rn(g * acc);
        if (st) {
#pragma unroll
            for (int k = 0; k < SP_MAX_TAPS - 1; ++k)
                if (k < hist) st[(size_t)k * H] = (k + 1 < hist) ? win[k + 1] : bx;
        }
    }
}

__device__ void sp_qk(const RvStepOp* op, SpShared* sh, int cta, int G, int wtid) {
    sp_row_scales(op, sh, wtid);
    const int lane = wtid & 31, w = wtid >> 5;
    const int nh = op->num_heads, nkv = op->num_kv_heads, hd = op->head_dim, half = hd >> 1;
    const int heads = nh + 2 * nkv;
    const size_t pstride = (size_t)SP_NPAD * op->N;
    for (int j = cta * 4 + w; j < op->M * heads; j += G * 4) {
        const int t = j / heads, h = j - t * heads;
        const float rs = sh->rs[t];
        const size_t row = (size_t)t * op->N + (size_t)h * hd;
        const bool is_q = h < nh, is_v = h >= nh + nkv;
        float a[4], b[4];                        // pairs (d, d + half), d = lane + 32 i
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int d = lane + 32 * i;
            a[i] = b[i] = 0.f;
            if (d < half) {
                a[i] = rs * sp_sum_parts(op->part, op->part_splits, pstride, row + d);
                b[i] = rs * sp_sum_parts(op->part, op->part_splits, pstride, row + half + d);
                ss += a[i] * a[i] + b[i] * b[i];
            }
        }
        ss = rv_warp_sum(ss);
        const int slot = is_q ? 0 : op->slot_mapping[t];
        if (!is_q && slot < 0) continue;
        const float* wv = is_q ? op->q_weight : op->k_weight;
        const float inv = (!is_v && wv) ? 1.f / sqrtf(ss / (float)hd + op->qk_eps) : 1.f;
        bf16* dst;
        if (is_q) dst = op->act_out + row;
        else if (!is_v) dst = op->k_cache + ((size_t)slot * nkv + (h - nh)) * hd;
        else dst = op->v_cache + ((size_t)slot * nkv + (h - nh - nkv)) * hd;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int d = lane + 32 * i;
            if (d >= half) continue;
            float x = a[i], y = b[i];
            if (!is_v) {
                if (wv) {
                    x = x * inv * wv[d];
                    y = y * inv * wv[half + d];
                }
                if (op->cos_table) {
                    const size_t trow = (size_t)op->positions[t] * half + d;
                    const float cs = op->cos_table[trow], sn = op->sin_table[trow];
                    const float xr = x * cs - y * sn, yr = x * sn + y * cs;
                    x = xr;
                    y = yr;
                }
            }
            dst[d] = __float2bfloat16_rn(x);
            dst[half + d] = __float2bfloat16_rn(y);
        }
    }
}

__device__ void sp_swiglu(const RvStepOp* op, SpShared* sh, int cta, int G, int wtid) {
    sp_row_scales(op, sh, wtid);
    const int F = op->N >> 1, F4 = F >> 2;          // F is a multiple of 8
    const size_t pstride = (size_t)SP_NPAD * op->N;
    for (int e = cta * SP_WORKERS + wtid; e < op->M * F4; e += G * SP_WORKERS) {
        const int t = e / F4, f = (e - t * F4) * 4;
        const float rs = sh->rs[t];
        const float* p = op->part + (size_t)t * op->N + f;
        float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
        for (int s = 0; s < op->part_splits; ++s) {
            const float4 a = *(const float4*)(p + s * pstride), b = *(const float4*)(p + s * pstride + F);
            g.x += a.x; g.y += a.y; g.z += a.z; g.w += a.w;
            u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
        }
        g.x *= rs; g.y *= rs; g.z *= rs; g.w *= rs;
        u.x *= rs; u.y *= rs; u.z *= rs; u.w *= rs;
        uint2 out;
        __nv_bfloat162* o2 = (__nv_bfloat162*)&out;
        o2[0] = __floats2bfloat162_rn(g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y);
        o2[1] = __floats2bfloat162_rn(g.z / (1.f + __expf(-g.z)) * u.z, g.w / (1.f + __expf(-g.w)) * u.w);
        *(uint2*)(op->act_out + (size_t)t * F + f) = out;
    }
}

__device__ void sp_logits(const RvStepOp* op, SpShared* sh, int cta, int G, int wtid) {
    sp_row_scales(op, sh, wtid);
    const int V = op->N;
    const size_t pstride = (size_t)SP_NPAD * V;
    if ((V & 3) == 0) {
        const int V4 = V >> 2;
        for (long long e = (long long)cta * SP_WORKERS + wtid; e < (long long)op->M * V4;
             e += (long long)G * SP_WORKERS) {
            const int t = (int)(e / V4), v = (int)(e - (long long)t * V4) * 4;
            const float rs = sh->rs[t];
            const float* p = op->part + (size_t)t * V + v;
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < op->part_splits; ++s) {
                const float4 b = *(const float4*)(p + s * pstride);
                a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
            }
            *(float4*)(op->logits + (size_t)t * V + v) = make_float4(a.x * rs, a.y * rs, a.z * rs, a.w * rs);
        }
    } else {
        for (long long e = (long long)cta * SP_WORKERS + wtid; e < (long long)op->M * V;
             e += (long long)G * SP_WORKERS) {
            const int t = (int)(e / V);
            op->logits[e] = sh->rs[t] * sp_sum_parts(op->part, op->part_splits, pstride, (size_t)e);
        }
    }
}

// ---- the kernel -----------------------------------------------------------------------------
__global__ void __launch_bounds__(SP_THREADS, 1)
step_program_kernel(const RvStepOp* __restrict__ ops, int n_ops, unsigned* counters, int* status,
                    int stages, unsigned long long* trace) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* ring = base;
    unsigned char* act = base + (size_t)stages * SP_W_BYTES;
    __shared__ SpShared sh;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, G = gridDim.x;
    // optional timeline of block 0 (eight stamps per operation), for measurements only
    unsigned long long* tr = (trace && cta == 0) ? trace : nullptr;
#define SP_STAMP(o, k) do { if (tr) tr[(o) * 8 + (k)] = sp_globaltimer(); } while (0)

    if (tid == 0) {
        sh.failed = 0;
        for (int s = 0; s < stages; ++s) {
            mbar_init(&sh.full_bar[s], 1);
            mbar_init(&sh.empty_bar[s], 1);
        }
        mbar_init(&sh.act_full, 1);
        mbar_init(&sh.act_free, 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sh.accum_full[b], 1);
            mbar_init(&sh.accum_empty[b], 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&sh.tmem_base)), "r"(32u));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = sh.tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer: weight tiles, as far ahead as the ring allows ------------------------
            long long it = 0;
            for (int o = 0; o < n_ops && !sh.failed; ++o) {
                const RvStepOp* op = ops + o;
                if (op->type != SP_GEMM) continue;
                int split, first, stride, kb0, kb1;
                if (!sp_items(op, cta, G, split, first, stride, kb0, kb1)) continue;
                for (int tile = first; tile < op->tiles && !sh.failed; tile += stride) {
                    for (int kb = kb0; kb < kb1; ++kb, ++it) {
                        const int s = (int)(it % stages);
                        if (it >= stages &&
                            !mbar_wait(&sh.empty_bar[s], (unsigned)((it / stages) - 1) & 1u, &sh.failed)) {
                            sp_fail(&sh, status, 31);
                            break;
                        }
                        mbar_expect_tx(&sh.full_bar[s], SP_W_BYTES);
                        tma_load_2d(ring + (size_t)s * SP_W_BYTES, &op->map_w, &sh.full_bar[s],
                                    kb * SP_BK, tile * SP_BM);
                    }
                }
            }
            // no copy of this block may still be in flight when it returns
            for (long long i = it > stages ? it - stages : 0; i < it; ++i) {
                const int s = (int)(i % stages);
                bool ok = false;
                const long long start = clock64();
                while (!ok && clock64() - start < RV_WAIT_CYCLES)
                    ok = mbar_try_wait(&sh.full_bar[s], (unsigned)(i / stages) & 1u);
                if (!ok) sp_fail(&sh, status, 32);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- the products: wait for inputs, copy the slice of x, issue the MMAs -------------
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                   ((unsigned)(SP_NPAD >> 3) << 17) | ((unsigned)(SP_BM >> 4) << 24);
            long long it = 0;
            unsigned acc_it = 0, act_loads = 0;
            for (int o = 0; o < n_ops && !sh.failed; ++o) {
                const RvStepOp* op = ops + o;
                if (op->type != SP_GEMM) continue;
                int split, first, stride, kb0, kb1;
                if (!sp_items(op, cta, G, split, first, stride, kb0, kb1)) continue;
                if (o > 0 && !sp_wait_done(counters + o - 1, (unsigned)G, &sh, status)) {
                    sp_fail(&sh, status, 35);
                    break;
                }
                SP_STAMP(o, 4);
                sp_fence_proxy_async();     // other blocks' stores (acquired above) before TMA reads
                if (act_loads > 0 && !mbar_wait(&sh.act_free, (act_loads - 1) & 1u, &sh.failed)) {
                    sp_fail(&sh, status, 34);
                    break;
                }
                const int nkb = kb1 - kb0;
                mbar_expect_tx(&sh.act_full, (unsigned)(nkb * SP_X_BYTES));
                for (int i = 0; i < nkb; ++i)
                    tma_load_2d(act + (size_t)i * SP_X_BYTES, &op->map_x, &sh.act_full,
                                (kb0 + i) * SP_BK, 0);
                if (!mbar_wait(&sh.act_full, act_loads & 1u, &sh.failed)) {
                    sp_fail(&sh, status, 34);
                    break;
                }
                ++act_loads;
                SP_STAMP(o, 5);
                for (int tile = first; tile < op->tiles && !sh.failed; tile += stride) {
                    const unsigned buf = acc_it & 1u;
                    if (acc_it >= 2 &&
                        !mbar_wait(&sh.accum_empty[buf], ((acc_it >> 1) - 1) & 1u, &sh.failed)) {
                        sp_fail(&sh, status, 37);
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned d = tmem_base + buf * SP_NPAD;
                    for (int i = 0; i < nkb; ++i, ++it) {
                        const int s = (int)(it % stages);
                        if (!mbar_wait(&sh.full_bar[s], (unsigned)(it / stages) & 1u, &sh.failed)) {
                            sp_fail(&sh, status, 33);
                            break;
                        }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const unsigned long long a0 = smem_desc_sw128(ring + (size_t)s * SP_W_BYTES);
                        const unsigned long long b0 = smem_desc_sw128(act + (size_t)i * SP_X_BYTES);
#pragma unroll
                        for (int k = 0; k < SP_BK / 16; ++k)
                            tcgen05_mma_f16(d, a0 + 2 * k, b0 + 2 * k, idesc, (i | k) != 0);
                        tcgen05_commit(&sh.empty_bar[s]);
                    }
                    if (sh.failed) break;
                    tcgen05_commit(&sh.accum_full[buf]);
                    ++acc_it;
                }
                tcgen05_commit(&sh.act_free);
                SP_STAMP(o, 6);
            }
        }
    } else {
        // ---- workers: accumulators to partial sums, and the elementwise operations --------------
        // The 128 workers meet at a named barrier, which has no time limit, so they must leave
        // the loop together: one thread samples `failed` before a barrier and all of them read
        // the sample after it.
        const int wtid = tid - 64;
        const unsigned lane_group = (unsigned)(warp & 3);      // the TMEM lanes this warp may read
        unsigned acc_it = 0;
        for (int o = 0; o < n_ops; ++o) {
            const RvStepOp* op = ops + o;
            const bool product = op->type == SP_GEMM;
            if (wtid == 0) {
                SP_STAMP(o, 0);
                if (!product && o > 0 && !sp_wait_done(counters + o - 1, (unsigned)G, &sh, status))
                    sp_fail(&sh, status, 35);
                sh.stop = sh.failed;
            }
            sp_worker_sync();
            if (sh.stop) break;
            if (wtid == 0) SP_STAMP(o, 1);
            if (product) {
                int split, first, stride, kb0, kb1;
                if (sp_items(op, cta, G, split, first, stride, kb0, kb1)) {
                    float* part = op->part + (size_t)split * SP_NPAD * op->N;
                    for (int tile = first; tile < op->tiles; tile += stride) {
                        const unsigned buf = acc_it & 1u;
                        int ok = 1;
                        if (lane == 0)
                            ok = mbar_wait(&sh.accum_full[buf], (acc_it >> 1) & 1u, &sh.failed) ? 1 : 0;
                        ok = __shfl_sync(0xffffffffu, ok, 0);
                        if (!ok) {
                            sp_fail(&sh, status, 36);
                            break;
                        }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        unsigned r[16];
                        tmem_load_16(tmem_base + ((lane_group * 32u) << 16) + buf * SP_NPAD, r);
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&sh.accum_empty[buf]);
                        const int n = tile * SP_BM + (int)lane_group * 32 + lane;
                        if (n < op->N) {
#pragma unroll
                            for (int t = 0; t < SP_NPAD; ++t)
                                if (t < op->M) part[(size_t)t * op->N + n] = __uint_as_float(r[t]);
                        }
                        ++acc_it;
                    }
                }
            } else {
                switch (op->type) {
                    case SP_RESID: sp_resid(op, cta, wtid); break;
                    case SP_CONV: sp_conv(op, &sh, cta, G, wtid); break;
                    case SP_QK: sp_qk(op, &sh, cta, G, wtid); break;
                    case SP_SWIGLU: sp_swiglu(op, &sh, cta, G, wtid); break;
                    case SP_LOGITS: sp_logits(op, &sh, cta, G, wtid); break;
                    default: break;
                }
            }
            // this block's share of operation o is done: make it visible, then count the block in
            if (wtid == 0) SP_STAMP(o, 2);
            __threadfence();
            sp_fence_proxy_async();
            sp_worker_sync();
            if (wtid == 0 && !sh.failed) {
                const unsigned old = atomicAdd(counters + o, 1u);
                if (old == (unsigned)G - 1) {
                    if (o > 0) counters[o - 1] = 0;          // nobody polls it any more
                    if (o == n_ops - 1) counters[o] = 0;     // nor this one: the list ends here
                }
                SP_STAMP(o, 3);
            }
        }
    }
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(32u));
    }
}

// ---- host side ---------------------------------------------------------------------------------
struct RvStepProgram {
    std::vector<RvStepOp> ops;
    RvStepOp* d_ops = nullptr;
    unsigned* d_counters = nullptr;
    int* status = nullptr;
    int grid = 0, stages = 0, finished = 0;
    unsigned long long* trace = nullptr;      // [ops][8] device timestamps of block 0, or null
    size_t smem = 0;
};

static int sp_env_int(const char* name, int fallback) {
    const char* e = getenv(name);
    return e && *e ? atoi(e) : fallback;
}

// How many K slices a product [N, K] is cut into on a grid of G blocks: as many as give every
// block an item in one round (G / tiles), at least what keeps a slice within SP_MAX_KB blocks.
// It depends on N, K and G only, so the order of a row's sum does not depend on the tokens.
extern "C" int rv_step_program_splits(int N, int K, int G) {
    const int tiles = (N + SP_BM - 1) / SP_BM, kb = (K + SP_BK - 1) / SP_BK;
    int s = G / (tiles > 0 ? tiles : 1);
    const int lo = (kb + SP_MAX_KB - 1) / SP_MAX_KB;
    if (s < lo) s = lo;
    if (s > kb) s = kb;
    if (s < 1) s = 1;
    return s;
}

extern "C" int rv_step_program_grid() { return sp_env_int("RVLLM_STEP_GRID", rv_sm_count()); }

extern "C" void* rv_step_program_create(int* status) {
    RvStepProgram* p = new (std::nothrow) RvStepProgram();
    if (!p) return nullptr;
    p->status = status;
    p->grid = rv_step_program_grid();
    p->stages = sp_env_int("RVLLM_STEP_STAGES", 11);
    if (p->stages > SP_MAX_STAGES) p->stages = SP_MAX_STAGES;
    if (p->stages < 2) p->stages = 2;
    p->smem = (size_t)p->stages * SP_W_BYTES + SP_ACT_BYTES + 1024;
    return p;
}

extern "C" void rv_step_program_destroy(void* handle) {
    RvStepProgram* p = (RvStepProgram*)handle;
    if (!p) return;
    if (p->d_ops) cudaFree(p->d_ops);
    if (p->d_counters) cudaFree(p->d_counters);
    delete p;
}

extern "C" int rv_step_program_len(void* handle) { return (int)((RvStepProgram*)handle)->ops.size(); }

static RvStepOp sp_blank(int type, int M) {
    RvStepOp op;
    memset(&op, 0, sizeof(op));
    op.type = type;
    op.M = M;
    return op;
}

#define SP_PROGRAM(handle)                                                           \
    RvStepProgram* p = (RvStepProgram*)(handle);                                     \
    if (!p || p->finished) RV_FAIL("step program: no program, or it is finished already")

// y = x . W^T into part [splits][16][N]; x is [16][K] bfloat16 (rows past M are never read for
// their values: they only have to exist), W [N][K] bfloat16.  Returns the number of slices in
// *splits_out.
extern "C" int rv_step_program_add_gemm(void* handle, const void* x, const void* w, float* part,
                                        int M, int N, int K, int* splits_out) {
    SP_PROGRAM(handle);
    if (M < 1 || M > SP_NPAD || N <= 0 || K <= 0) RV_FAIL("step program: product sizes out of range");
    if (K % 8) RV_FAIL("step program: K = %d must be a multiple of 8", K);
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)part) % 16) RV_FAIL("step program: operands must be 16-byte aligned");
    RvStepOp op = sp_blank(SP_GEMM, M);
    op.N = N;
    op.K = K;
    op.tiles = (N + SP_BM - 1) / SP_BM;
    op.kblocks = (K + SP_BK - 1) / SP_BK;
    op.splits = rv_step_program_splits(N, K, p->grid);
    if (op.splits > p->grid) RV_FAIL("step program: K = %d needs %d slices but the grid has %d blocks", K, op.splits, p->grid);
    op.part = part;
    if (make_map(&op.map_w, w, N, K, SP_BM)) return 1;
    if (make_map(&op.map_x, x, SP_NPAD, K, SP_NPAD)) return 1;
    p->ops.push_back(op);
    if (splits_out) *splits_out = op.splits;
    return 0;
}

static void sp_set_scale(RvStepOp& op, const float* ss_in, int n_slices, float eps, float dim) {
    op.ss_in = ss_in;
    op.n_slices = ss_in ? n_slices : 0;
    op.eps = eps;
    op.dim = dim;
}

// stream [16][H] += sum of `part_splits` slices of part (+ bias), or = embed[token_ids] * scale;
// xw = bfloat16(stream * w_next); ss_out [ceil(H / 64)][16] sums of squares by column slice.
extern "C" int rv_step_program_add_resid(void* handle, float* resid, const float* part, int part_splits,
                                         const float* bias, const void* embed, const int* token_ids,
                                         float embed_scale, int vocab, const float* w_next, void* xw,
                                         float* ss_out, int M, int H) {
    SP_PROGRAM(handle);
    if (H % 8) RV_FAIL("step program: width %d must be a multiple of 8", H);
    if ((H + SP_SLICE - 1) / SP_SLICE > p->grid) RV_FAIL("step program: width %d exceeds the grid", H);
    if (!embed && (!part || part_splits < 1)) RV_FAIL("step program: nothing to add to the stream");
    RvStepOp op = sp_blank(SP_RESID, M);
    op.N = H;
    op.resid = resid;
    op.part = (float*)part;
    op.part_splits = part_splits;
    op.bias = bias;
    op.embed = (const bf16*)embed;
    op.token_ids = token_ids;
    op.embed_scale = embed_scale;
    op.vocab = vocab;
    op.w_next = w_next;
    op.xw = (bf16*)xw;
    op.ss_out = ss_out;
    p->ops.push_back(op);
    return 0;
}

extern "C" int rv_step_program_add_conv(void* handle, const float* part, int part_splits,
                                        const float* ss_in, int n_slices, float eps, float dim,
                                        const float* filter, const float* in_bias,
                                        const float* conv_bias, float* state, const int* state_slot,
                                        const int* start_pos, void* act_out, int M, int hidden,
                                        int taps) {
    SP_PROGRAM(handle);
    if (taps < 1 || taps > SP_MAX_TAPS) RV_FAIL("step program: filter length %d is not supported", taps);
    RvStepOp op = sp_blank(SP_CONV, M);
    op.N = 3 * hidden;
    op.part = (float*)part;
    op.part_splits = part_splits;
    sp_set_scale(op, ss_in, n_slices, eps, dim);
    op.filter = filter;
    op.in_bias = in_bias;
    op.conv_bias = conv_bias;
    op.state = state;
    op.state_slot = state_slot;
    op.start_pos = start_pos;
    op.act_out = (bf16*)act_out;
    op.hidden = hidden;
    op.taps = taps;
    p->ops.push_back(op);
    return 0;
}

extern "C" int rv_step_program_add_qk(void* handle, const float* part, int part_splits,
                                      const float* ss_in, int n_slices, float eps, float dim,
                                      int num_heads, int num_kv_heads, int head_dim,
                                      const float* q_weight, const float* k_weight, float qk_eps,
                                      const float* cos_table, const float* sin_table,
                                      const int* positions, const int* slot_mapping, void* k_cache,
                                      void* v_cache, void* q_out, int M) {
    SP_PROGRAM(handle);
    if (head_dim % 2 || head_dim > 256) RV_FAIL("step program: head size %d is not supported", head_dim);
    if (num_kv_heads > 0 && (!k_cache || !v_cache || !slot_mapping))
        RV_FAIL("step program: key/value heads given without a cache to write");
    RvStepOp op = sp_blank(SP_QK, M);
    op.N = (num_heads + 2 * num_kv_heads) * head_dim;
    op.part = (float*)part;
    op.part_splits = part_splits;
    sp_set_scale(op, ss_in, n_slices, eps, dim);
    op.num_heads = num_heads;
    op.num_kv_heads = num_kv_heads;
    op.head_dim = head_dim;
    op.q_weight = q_weight;
    op.k_weight = k_weight;
    op.qk_eps = qk_eps;
    op.cos_table = cos_table;
    op.sin_table = sin_table;
    op.positions = positions;
    op.slot_mapping = slot_mapping;
    op.k_cache = (bf16*)k_cache;
    op.v_cache = (bf16*)v_cache;
    op.act_out = (bf16*)q_out;
    p->ops.push_back(op);
    return 0;
}

extern "C" int rv_step_program_add_swiglu(void* handle, const float* part, int part_splits,
                                          const float* ss_in, int n_slices, float eps, float dim,
                                          void* act_out, int M, int ffn) {
    SP_PROGRAM(handle);
    if (ffn % 8) RV_FAIL("step program: feed-forward width %d must be a multiple of 8", ffn);
    RvStepOp op = sp_blank(SP_SWIGLU, M);
    op.N = 2 * ffn;
    op.part = (float*)part;
    op.part_splits = part_splits;
    sp_set_scale(op, ss_in, n_slices, eps, dim);
    op.act_out = (bf16*)act_out;
    p->ops.push_back(op);
    return 0;
}

extern "C" int rv_step_program_add_logits(void* handle, const float* part, int part_splits,
                                          const float* ss_in, int n_slices, float eps, float dim,
                                          float* logits, int M, int vocab) {
    SP_PROGRAM(handle);
    RvStepOp op = sp_blank(SP_LOGITS, M);
    op.N = vocab;
    op.part = (float*)part;
    op.part_splits = part_splits;
    sp_set_scale(op, ss_in, n_slices, eps, dim);
    op.logits = logits;
    p->ops.push_back(op);
    return 0;
}

// Upload the list.  Call it outside any stream capture (it allocates and copies).
extern "C" int rv_step_program_finish(void* handle) {
    SP_PROGRAM(handle);
    if (p->ops.empty()) RV_FAIL("step program: the list is empty");
    cudaError_t e = cudaFuncSetAttribute(step_program_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)p->smem);
    if (e != cudaSuccess) RV_FAIL("step program: %s", cudaGetErrorString(e));
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, step_program_kernel, SP_THREADS, p->smem);
    if (e != cudaSuccess) RV_FAIL("step program: %s", cudaGetErrorString(e));
    if (per_sm < 1 || p->grid > per_sm * rv_sm_count())
        RV_FAIL("step program: %d blocks cannot all be resident on this device", p->grid);
    const size_t bytes = p->ops.size() * sizeof(RvStepOp);
    e = cudaMalloc((void**)&p->d_ops, bytes);
    if (e == cudaSuccess) e = cudaMalloc((void**)&p->d_counters, p->ops.size() * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMemcpy(p->d_ops, p->ops.data(), bytes, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemset(p->d_counters, 0, p->ops.size() * sizeof(unsigned));
    if (e != cudaSuccess) RV_FAIL("step program: %s", cudaGetErrorString(e));
    p->finished = 1;
    return 0;
}

// Operations [first, first + count) as one cooperative launch.  The counters are zero before
// and after a launch that ran to its end; after a launch that set `status` call
// rv_step_program_reset before the next one.
extern "C" int rv_step_program_run(void* handle, int first, int count, void* stream) {
    RvStepProgram* p = (RvStepProgram*)handle;
    if (!p || !p->finished) RV_FAIL("step program: not finished");
    if (first < 0 || count < 1 || first + count > (int)p->ops.size()) RV_FAIL("step program: bad range");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p->grid, 1, 1);
    cfg.blockDim = dim3(SP_THREADS, 1, 1);
    cfg.dynamicSmemBytes = p->smem;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const RvStepOp* ops = p->d_ops + first;
    unsigned* counters = p->d_counters + first;
    unsigned long long* trace = p->trace ? p->trace + (size_t)first * 8 : nullptr;
    cudaError_t e = cudaLaunchKernelEx(&cfg, step_program_kernel, ops, count, counters, p->status,
                                       p->stages, trace);
    if (e != cudaSuccess) RV_FAIL("step program: %s", cudaGetErrorString(e));
    return 0;
}

// For measurements: block 0 writes eight %globaltimer stamps per operation into `trace`
// ([operations][8] 64-bit words of device memory; null switches it off again): worker leader at
// the operation's start, after its inputs are ready, after its work, after it counted itself in;
// for products also the issuing thread after its inputs are ready, after its slice of x has
// arrived, after its last MMA was issued.
extern "C" int rv_step_program_trace(void* handle, unsigned long long* trace) {
    RvStepProgram* p = (RvStepProgram*)handle;
    if (!p) RV_FAIL("step program: no program");
    p->trace = trace;
    return 0;
}

extern "C" int rv_step_program_reset(void* handle, void* stream) {
    RvStepProgram* p = (RvStepProgram*)handle;
    if (!p || !p->finished) RV_FAIL("step program: not finished");
    cudaError_t e = cudaMemsetAsync(p->d_counters, 0, p->ops.size() * sizeof(unsigned), (cudaStream_t)stream);
    if (e != cudaSuccess) RV_FAIL("step program: %s", cudaGetErrorString(e));
    return 0;
}
