// Weight-streaming matrix product for few tokens on the 5th-generation tensor cores:
//   y[M, N] = x[M, K] . W[N, K]^T,  bfloat16 operands, float32 accumulation,
// for M <= 256 tokens (decode steps and short prompt portions), where the product is
// bound by reading W once from HBM.
//
// The roles are swapped with respect to the usual orientation: 128 rows of W are the M
// side of a tcgen05.mma (cta_group::1, M = 128, kind::f16) and the tokens, padded to a
// multiple of 16, are its N side, so one instruction covers 128 output columns for all
// tokens and the accumulator [128 lanes x tokens] lives in TMEM.  Operands reach shared
// memory by TMA (cp.async.bulk.tensor.2d, 128-byte swizzle, K-major tiles of 64
// elements) through a ring of stages guarded by mbarriers; one elected thread issues the
// copies, one issues the MMAs (four K = 16 steps per stage), tcgen05.commit hands a
// stage back to the producer, and after the last stage the four warps read the
// accumulator with tcgen05.ld and write y.  The K range is split over the blocks of a
// thread-block cluster (1, 2, 4 or 8 of them) so that every SM streams a share of W; each
// block parks its float32 partial tile in its own shared memory, the cluster meets at a
// barrier, and block r adds, for the tokens t = r mod size, the partial rows of all blocks
// in rank order through distributed shared memory (no atomics, no global workspace: the
// sum is deterministic).  The TMA copies are per block: no multicast.
//
// Every wait on an mbarrier is bounded: after RV_WAIT_CYCLES clock cycles the thread
// records an error code in `status`, every role leaves its loop, the producer waits
// (again bounded) for the copies it has in flight, TMEM is freed and the block returns.
//
// Reference counterpart: `linear_f16` = cublasGemmEx (src/cuda/cublas_ops.rs:44-92).
// Plain reference: tests/plain_ops.py linear.
#include "tcgen05_common.cuh"

#define RV_GEMM_BM 128          // rows of W per block (the MMA's M)
#define RV_GEMM_BK 64           // K elements per stage: 128 bytes, one swizzle row
#define RV_GEMM_MAX_STAGES 12
#define RV_GEMM_SMEM_LIMIT (226 * 1024)

// ---- the kernel -----------------------------------------------------------------------
// grid (n_tiles, splits) with clusters of (1, splits); block 128 threads.
// status[0]: first error code (0 = none).
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The same meeting without memory ordering: it only keeps every block alive until all have
// finished reading the others' shared memory (a release here would first wait for the
// output stores just issued).
__device__ __forceinline__ void cluster_sync_relaxed() {
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(const float* local, unsigned rank) {
    unsigned remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

// What the q|k|v product's epilogue needs to finish the job of the q/k norm + rotation + cache
// write kernel (head size 64: a tile of 128 weight rows is two whole heads).
struct RvQkvEpilogue {
    const float* q_weight;        // [64] or null
    const float* k_weight;        // [64] or null
    const float* cos_table;       // [positions, 32] or null (no rotation)
    const float* sin_table;
    const int* positions;         // [tokens]
    const int* slot_mapping;      // [tokens]: page * page_size + offset, or -1
    bf16* k_cache;                // [slots, kv_heads, 64]
    bf16* v_cache;
    float eps;
    int num_heads, num_kv_heads;
};

// QKV = false: y = x . W^T.  QKV = true (bfloat16 output, up to 16 tokens, head size 64): W is
// the q|k|v projection; the sums are rounded to bfloat16 as they would be stored, then each
// query and key head is RMS-normalised and rotated, queries go to `out`, keys and values to
// their slots of the paged cache: the separate kernel for that, and its place in the chain of
// dependent launches, are gone.
// A plain product carries no epilogue arguments at all.
struct RvNoEpilogue {};
template <bool QKV> struct RvEpilogueOf { typedef RvNoEpilogue type; };
template <> struct RvEpilogueOf<true> { typedef RvQkvEpilogue type; };

template <typename TO, bool QKV, int KBS>
__global__ void __launch_bounds__(128) gemm_tcgen05_kernel(
    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
    TO* __restrict__ out, int* __restrict__ status, int M, int N, int kblocks, int n_pad,
    int stages, const typename RvEpilogueOf<QKV>::type epi, const bf16* __restrict__ w_tiled) {
    constexpr int kbs = KBS;          // K blocks of 64 per stage
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // the dynamic segment is aligned by hand: swizzled tiles need 1024-byte alignment
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // a stage holds `kbs` K blocks of 64: kbs weight tiles of 16 KB (one contiguous copy when
    // the matrix is laid out tile by tile) and kbs x tiles
    const int w_tile = RV_GEMM_BM * RV_GEMM_BK * 2, x_tile = n_pad * RV_GEMM_BK * 2;
    const int w_bytes = kbs * w_tile;
    const int x_bytes = kbs * x_tile;
    unsigned char* w_tiles = base;
    unsigned char* x_tiles = base + stages * w_bytes;
    __shared__ __align__(8) unsigned long long full_bar[RV_GEMM_MAX_STAGES];
    __shared__ __align__(8) unsigned long long empty_bar[RV_GEMM_MAX_STAGES];
    __shared__ __align__(8) unsigned long long accum_bar;
    __shared__ unsigned tmem_base_smem;
    __shared__ volatile int failed;

    // The next kernel of the stream may start its own preamble now.  This kernel's wait
    // for the previous one comes later: W does not depend on it, only x and y do.
    rv_pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x, split = blockIdx.y, splits = gridDim.y;
    const int kb0 = (int)((long long)kblocks * split / splits);
    const int kb1 = (int)((long long)kblocks * (split + 1) / splits);
    const int nkb = kb1 - kb0;
    const int nst = (nkb + kbs - 1) / kbs;             // stages' worth of work
    unsigned tmem_cols = 32;
    while ((int)tmem_cols < n_pad) tmem_cols <<= 1;

    if (tid == 0) {
        failed = 0;
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_smem)), "r"(tmem_cols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = tmem_base_smem;

    if (warp == 0 && lane == 0) {
        // ---- producer: TMA copies of W and x tiles ------------------------------------
        // The weight tiles of a stage come as one contiguous bulk copy when the matrix was laid
        // out tile by tile beforehand (`rv_gemm_tile_weights`; an SM copies 32 KB at a time more
        // than twice as fast as tensor-map boxes of 128 strided rows), else as tensor-map boxes.
        auto blocks_of = [&](int i) { return min(kbs, nkb - i * kbs); };
        auto load_w = [&](int s, int i) {
            const int kb = kb0 + i * kbs, cnt = blocks_of(i);
            mbar_expect_tx(&full_bar[s], (unsigned)(cnt * (w_tile + x_tile)));
            if (w_tiled) {
                bulk_load_1d(w_tiles + s * w_bytes,
                             w_tiled + ((size_t)tile * kblocks + kb) * (RV_GEMM_BM * RV_GEMM_BK),
                             (unsigned)(cnt * w_tile), &full_bar[s]);
            } else {
#pragma unroll
                for (int j = 0; j < kbs; ++j)
                    if (j < cnt)
                        tma_load_2d(w_tiles + s * w_bytes + j * w_tile, &map_w, &full_bar[s],
                                    (kb + j) * RV_GEMM_BK, tile * RV_GEMM_BM);
            }
        };
        auto load_x = [&](int s, int i) {
            const int kb = kb0 + i * kbs, cnt = blocks_of(i);
#pragma unroll
            for (int j = 0; j < kbs; ++j)
                if (j < cnt)
                    tma_load_2d(x_tiles + s * x_bytes + j * x_tile, &map_x, &full_bar[s],
                                (kb + j) * RV_GEMM_BK, 0);
        };
        // fill the ring with weight tiles before waiting for the previous kernel: they
        // stream from HBM while it is still running
        const int pre = min(nst, stages);
        for (int i = 0; i < pre; ++i) load_w(i, i);
        rv_pdl_wait();
        for (int i = 0; i < pre; ++i) load_x(i, i);
        int issued = pre;
        for (int i = pre; i < nst; ++i) {
            const int s = i % stages;
            {
                const unsigned parity = ((i / stages) - 1) & 1;
                if (!mbar_wait(&empty_bar[s], parity, &failed)) {
                    if (!failed) { failed = 1; atomicCAS(status, 0, 1); }
                    break;
                }
            }
            load_w(s, i);
            load_x(s, i);
            issued = i + 1;
        }
        // no copy of this block may still be in flight when it returns
        for (int i = max(0, issued - stages); i < issued; ++i) {
            const int s = i % stages;
            bool ok = false;
            const long long start = clock64();
            while (!ok && clock64() - start < RV_WAIT_CYCLES)
                ok = mbar_try_wait(&full_bar[s], (i / stages) & 1);
            if (!ok && !failed) { failed = 1; atomicCAS(status, 0, 2); }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer -------------------------------------------------------------------
        rv_pdl_wait();     // the bounded waits below start only when the previous kernel is done
        // instruction descriptor: D float32, A and B bfloat16, both K-major, N = n_pad, M = 128
        const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                               ((unsigned)(n_pad >> 3) << 17) | ((unsigned)(RV_GEMM_BM >> 4) << 24);
        for (int i = 0; i < nst; ++i) {
            const int s = i % stages;
            if (!mbar_wait(&full_bar[s], (i / stages) & 1, &failed)) {
                if (!failed) { failed = 1; atomicCAS(status, 0, 3); }
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int cnt = min(kbs, nkb - i * kbs);
#pragma unroll
            for (int j = 0; j < kbs; ++j) {
                if (j >= cnt) break;
                const unsigned long long a0 = smem_desc_sw128(w_tiles + s * w_bytes + j * w_tile);
                const unsigned long long b0 = smem_desc_sw128(x_tiles + s * x_bytes + j * x_tile);
#pragma unroll
                for (int k = 0; k < RV_GEMM_BK / 16; ++k)      // 32 bytes per K = 16 step
                    tcgen05_mma_f16(tmem_base, a0 + 2 * k, b0 + 2 * k, idesc, (i | j | k) != 0);
            }
            tcgen05_commit(&empty_bar[s]);                  // frees the stage when the MMAs are done
        }
        tcgen05_commit(&accum_bar);                         // arrives when every MMA above is done
        // this thread alone polls for the accumulator; the other 127 sleep at the block
        // barrier below instead of competing with the two working threads for issue slots
        if (!failed && !mbar_wait(&accum_bar, 0, &failed) && !failed) {
            failed = 1;
            atomicCAS(status, 0, 4);
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncwarp();
    rv_pdl_wait();            // before any thread writes y: the previous kernel is done

    // ---- epilogue: all four warps, warp w owns TMEM lanes [32w, 32w + 32) -------------------
    __syncthreads();          // the accumulator is complete, `failed` is final, the producer
                              // has drained its copies
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const bool good = !failed;
    const int n_local = warp * 32 + lane;
    const int n = tile * RV_GEMM_BM + n_local;                // this thread's output column
    float* park = (float*)base;                               // [token][128], over the stage ring
    for (int c = 0; c < n_pad; c += 16) {
        unsigned r[16];
        tmem_load_16(tmem_base + ((unsigned)(warp * 32) << 16) + (unsigned)c, r);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int t = c + j;
            if (t < M) {
                const float v = good ? __uint_as_float(r[j]) : 0.f;
                if (splits == 1 && !QKV) {
                    if (n < N && good) rv_store(out + (size_t)t * N + n, v);
                } else {
                    park[t * RV_GEMM_BM + n_local] = v;
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(tmem_cols));
    }
    if constexpr (QKV) {
        // ---- q|k|v: this block finishes its tokens (t = split, split + splits, ...) ------------
        __shared__ float red[4];
        __shared__ float xs[RV_GEMM_BM];
        if (splits > 1) cluster_sync_all();                   // all partial tiles are parked
        const int hcol = n >> 6, d = n & 63, lh = n_local >> 6;
        const int kind = hcol < epi.num_heads ? 0 : (hcol < epi.num_heads + epi.num_kv_heads ? 1 : 2);
        const float* wv = kind == 0 ? epi.q_weight : epi.k_weight;
        const bool normed = kind < 2 && wv != nullptr && n < N;
        const float wgt = normed ? wv[d] : 1.f;
        for (int t = split; t < M; t += splits) {
            float acc = 0.f;
            for (int s = 0; s < splits; ++s)
                acc += ld_cluster_f32(park + t * RV_GEMM_BM + n_local, (unsigned)s);
            const float x = __bfloat162float(__float2bfloat16_rn(acc));   // as it would be stored
            const int slot = epi.slot_mapping[t];
            float c = 1.f, sn = 0.f;
            if (kind < 2 && epi.cos_table && n < N) {
                const size_t trow = (size_t)epi.positions[t] * 32 + (d & 31);
                c = epi.cos_table[trow];
                sn = epi.sin_table[trow];
            }
            const float ss_w = rv_warp_sum(x * x);
            if (lane == 0) red[warp] = ss_w;
            __syncthreads();
            float xn = x;
            if (normed) xn = x / sqrtf((red[2 * lh] + red[2 * lh + 1]) / 64.f + epi.eps) * wgt;
            xs[n_local] = xn;
            __syncthreads();
            float res = xn;
            if (kind < 2 && epi.cos_table) {
                const float other = xs[n_local ^ 32];         // dimension d + 32 or d - 32
                res = d < 32 ? xn * c - other * sn : other * sn + xn * c;
            }
            if (n < N && good) {
                if (kind == 0) {
                    rv_store(out + (size_t)t * N + n, res);
                } else if (slot >= 0) {
                    bf16* cache = kind == 1 ? epi.k_cache : epi.v_cache;
                    const int hh = hcol - epi.num_heads - (kind == 2 ? epi.num_kv_heads : 0);
                    cache[((size_t)slot * epi.num_kv_heads + hh) * 64 + d] = __float2bfloat16_rn(res);
                }
            }
            __syncthreads();                                  // red and xs are used again
        }
        if (splits > 1) cluster_sync_relaxed();               // nobody leaves while it is read
        return;
    }
    if (splits == 1) return;

    // ---- every block of the cluster adds its share of token rows, in rank order ----------
    cluster_sync_all();                                       // all partial tiles are parked
    if (n < N) {
        for (int t = split; t < M; t += splits) {
            float acc = 0.f;
            for (int s = 0; s < splits; ++s)
                acc += ld_cluster_f32(park + t * RV_GEMM_BM + n_local, (unsigned)s);
            rv_store(out + (size_t)t * N + n, acc);
        }
    }
    cluster_sync_relaxed();                                   // nobody leaves while it is read
}

static int env_int(const char* name, int fallback) {
    const char* e = getenv(name);
    return e && *e ? atoi(e) : fallback;
}

// How many blocks (1 to 8, the portable cluster size) share the K range of one tile: doubled
// until there is about one block per SM, as long as each keeps at least four stages of work.
// (RVLLM_GEMM_POW2=0 selects a wave-cost model instead; timed on the LFM2-1.2B decode step
// it was a few per cent slower.)  The split depends on N and K only, so the order of a row's
// sum does not depend on how many tokens share the launch.
extern "C" int rv_gemm_tcgen05_splits(int N, int K) {
    const int tiles = (N + RV_GEMM_BM - 1) / RV_GEMM_BM;
    const int kblocks = (K + RV_GEMM_BK - 1) / RV_GEMM_BK;
    static int forced = env_int("RVLLM_GEMM_SPLITS", 0);
    static int fixed_cost = env_int("RVLLM_GEMM_FIXED", 6);
    static int sms = env_int("RVLLM_GEMM_SLOTS", 3 * rv_sm_count());
    if (forced > 0) return forced > 8 ? 8 : (kblocks / forced < 1 ? 1 : forced);
    static int pow2 = env_int("RVLLM_GEMM_POW2", 1);
    if (pow2) {        // doubling until about one block per SM, at least four stages each
        int s = 1;
        // RVLLM_GEMM_MINBLOCKS: measured in the LFM2-1.2B decode step at batch 8: 128 (gate|up
        // unsplit) 0.973 ms, 148 (one block per SM, the default) 0.947 ms, 222 0.985 ms, 296 1.062 ms
        static int min_blocks = env_int("RVLLM_GEMM_MINBLOCKS", rv_sm_count());
        while (s < 8 && tiles * s < min_blocks && kblocks / (2 * s) >= 4) s *= 2;
        return s;
    }
    int best = 1;
    long long best_cost = -1;
    for (int s = 1; s <= 8; ++s) {
        if (s > 1 && kblocks / s < 2) break;
        const long long waves = ((long long)tiles * s + sms - 1) / sms;
        const long long cost = waves * ((kblocks + s - 1) / s + fixed_cost);
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best = s;
        }
    }
    return best;
}

// Stages of the copy ring.  Six by default (108 KB with 16 tokens): two blocks fit an SM, so
// the next kernel's blocks can already fill their rings while this one computes; deeper
// rings that leave room for one block per SM measured much slower.
static int pick_stages(int n_pad, int kbs) {
    static int want1 = env_int("RVLLM_GEMM_STAGES", 6);
    static int want_wide = env_int("RVLLM_GEMM_STAGES_WIDE", 4);
    const int want = kbs > 1 ? (want1 + kbs - 1) / kbs : want1;      // the same ring in bytes
    const int per_stage = kbs * (RV_GEMM_BM * RV_GEMM_BK * 2 + n_pad * RV_GEMM_BK * 2);
    int st = (RV_GEMM_SMEM_LIMIT - 1024) / per_stage;
    // More than 16 tokens: stages are larger, and four of them keep two blocks on an SM (a
    // deeper ring copies no faster: an SM's copy rate does not grow beyond four stages)
    const int cap = n_pad > 16 ? want_wide : want;
    if (st > cap) st = cap;
    return st > RV_GEMM_MAX_STAGES ? RV_GEMM_MAX_STAGES : st;
}

// Once per process, outside any stream capture: raise the kernels' shared-memory limit and
// look up the driver's tensor-map encoder.
template <typename TO, bool QKV, int KBS>
static cudaError_t raise_smem() {
    return cudaFuncSetAttribute(gemm_tcgen05_kernel<TO, QKV, KBS>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize, RV_GEMM_SMEM_LIMIT);
}

extern "C" int rv_gemm_tcgen05_init() {
    cudaError_t e = raise_smem<bf16, false, 1>();
    if (e == cudaSuccess) e = raise_smem<bf16, false, 2>();
    if (e == cudaSuccess) e = raise_smem<bf16, false, 3>();
    if (e == cudaSuccess) e = raise_smem<float, false, 1>();
    if (e == cudaSuccess) e = raise_smem<float, false, 2>();
    if (e == cudaSuccess) e = raise_smem<float, false, 3>();
    if (e == cudaSuccess) e = raise_smem<bf16, true, 1>();
    if (e == cudaSuccess) e = raise_smem<bf16, true, 2>();
    if (e == cudaSuccess) e = raise_smem<bf16, true, 3>();
    if (e != cudaSuccess) RV_FAIL("gemm_tcgen05: %s", cudaGetErrorString(e));
    if (!encode_fn()) RV_FAIL("gemm_tcgen05: cuTensorMapEncodeTiled is not available in this driver");
    return 0;
}

template <bool QKV> static typename RvEpilogueOf<QKV>::type pass_epi(const RvQkvEpilogue& e);
template <> RvNoEpilogue pass_epi<false>(const RvQkvEpilogue&) { return RvNoEpilogue{}; }
template <> RvQkvEpilogue pass_epi<true>(const RvQkvEpilogue& e) { return e; }

template <typename TO, bool QKV, int KBS>
static int launch_kbs(const CUtensorMap& map_w, const CUtensorMap& map_x, void* out, int* status, int M,
                  int N, int kblocks, int n_pad, int stages, int tiles, int splits, size_t smem,
                  const RvQkvEpilogue& epi, const void* w_tiled, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles, splits, 1);
    cfg.blockDim = dim3(128, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = splits;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = rv_pdl_enabled();
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<TO, QKV, KBS>, map_w, map_x, (TO*)out,
                                       status, M, N, kblocks, n_pad, stages, pass_epi<QKV>(epi), (const bf16*)w_tiled);
    if (e != cudaSuccess) RV_FAIL("gemm_tcgen05: %s", cudaGetErrorString(e));
    return 0;
}

template <typename TO, bool QKV>
static int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, void* out, int* status, int M,
                  int N, int kblocks, int n_pad, int stages, int tiles, int splits, size_t smem,
                  const RvQkvEpilogue& epi, const void* w_tiled, int kbs, cudaStream_t stream) {
    if (kbs == 3)
        return launch_kbs<TO, QKV, 3>(map_w, map_x, out, status, M, N, kblocks, n_pad, stages, tiles,
                                      splits, smem, epi, w_tiled, stream);
    if (kbs == 2)
        return launch_kbs<TO, QKV, 2>(map_w, map_x, out, status, M, N, kblocks, n_pad, stages, tiles,
                                      splits, smem, epi, w_tiled, stream);
    return launch_kbs<TO, QKV, 1>(map_w, map_x, out, status, M, N, kblocks, n_pad, stages, tiles,
                                  splits, smem, epi, w_tiled, stream);
}

// y = x . W^T.  `status` is a device int the kernel sets to a non-zero code if a bounded
// wait ran out (1: producer waiting for a free stage, 2: copies still in flight at exit,
// 3: MMA issuer waiting for data, 4: epilogue waiting for the accumulator).
static int gemm(const void* x, const void* w, void* out, int out_dtype, int* status, int M, int N,
                int K, const RvQkvEpilogue* epi, const void* w_tiled, void* stream) {
    if (M == 0) return 0;
    if (M < 0 || M > 256 || N <= 0 || K <= 0)
        RV_FAIL("gemm_tcgen05: sizes out of range (M = %d must be 1..256, N = %d, K = %d)", M, N, K);
    if (K % 8) RV_FAIL("gemm_tcgen05: K = %d must be a multiple of 8 (16-byte rows for TMA)", K);
    if (((uintptr_t)x | (uintptr_t)w) % 16) RV_FAIL("gemm_tcgen05: operands must be 16-byte aligned");
    const int n_pad = ((M + 15) / 16) * 16;
    const int tiles = (N + RV_GEMM_BM - 1) / RV_GEMM_BM;
    const int kblocks = (K + RV_GEMM_BK - 1) / RV_GEMM_BK;
    const int splits = rv_gemm_tcgen05_splits(N, K);
    // K blocks per stage: two (copies of 32 KB) for a matrix laid out tile by tile and few tokens
    static int kbs_tiled = env_int("RVLLM_GEMM_STAGE_BLOCKS", 2);
    // (with more tokens the larger stages measured slower: 64 tokens 15 - 30 us a product with one
    // block a stage, 17 - 37 with two, cuBLAS 5 - 14)
    const int kbs = (w_tiled && n_pad <= 16 && (kbs_tiled == 2 || kbs_tiled == 3)) ? kbs_tiled : 1;
    const int stages = pick_stages(n_pad, kbs);
    const size_t ring = (size_t)stages * kbs * (RV_GEMM_BM * RV_GEMM_BK * 2 + n_pad * RV_GEMM_BK * 2);
    if (stages < 2) RV_FAIL("gemm_tcgen05: no room for two stages with %d tokens", M);
    if (splits > 1 && (size_t)M * RV_GEMM_BM * 4 > ring)
        RV_FAIL("gemm_tcgen05: the partial tile of %d tokens does not fit the stage ring", M);
    CUtensorMap map_w, map_x;
    if (make_map(&map_w, w, N, K, RV_GEMM_BM)) return 1;
    if (make_map(&map_x, x, M, K, n_pad)) return 1;
    const size_t smem = ring + 1024;
    cudaStream_t s = (cudaStream_t)stream;
    const RvQkvEpilogue none = {};
    if (epi) {
        if (out_dtype != RV_DTYPE_BF16 || M > 16)
            RV_FAIL("gemm_tcgen05: the q|k|v epilogue takes bfloat16 and up to 16 tokens");
        return launch<bf16, true>(map_w, map_x, out, status, M, N, kblocks, n_pad, stages, tiles, splits,
                                  smem, *epi, w_tiled, kbs, s);
    }
    if (out_dtype == RV_DTYPE_BF16)
        return launch<bf16, false>(map_w, map_x, out, status, M, N, kblocks, n_pad, stages, tiles, splits,
                                   smem, none, w_tiled, kbs, s);
    if (out_dtype == RV_DTYPE_F32)
        return launch<float, false>(map_w, map_x, out, status, M, N, kblocks, n_pad, stages, tiles,
                                    splits, smem, none, w_tiled, kbs, s);
    RV_FAIL("gemm_tcgen05: unknown output dtype code %d", out_dtype);
}

// `w_tiled` (may be null): the same matrix as written by rv_gemm_tile_weights.
extern "C" int rv_gemm_tcgen05(const void* x, const void* w, void* out, int out_dtype, int* status,
                               int M, int N, int K, const void* w_tiled, void* stream) {
    return gemm(x, w, out, out_dtype, status, M, N, K, nullptr, w_tiled, stream);
}

// The weight matrix laid out for contiguous copies: tile (t, kb) = rows [128 t, 128 t + 128) x
// columns [64 kb, 64 kb + 64) of W [N, K] as the 16 KB image the MMA reads from shared memory
// (rows of 128 bytes whose 16-byte chunks are XOR-swizzled with the row index mod 8), tiles in
// (t, kb) order, rows and columns past the matrix as zeros.
__global__ void tile_weights_kernel(const bf16* __restrict__ w, uint4* __restrict__ out, int N, int K,
                                    int kblocks, long long chunks) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < chunks;
         i += (long long)gridDim.x * blockDim.x) {
        const int ch = (int)(i & 7), r = (int)((i >> 3) & 127);
        const long long tile_kb = i >> 10;                       // 1024 chunks of 16 bytes per tile
        const int kb = (int)(tile_kb % kblocks);
        const long long t = tile_kb / kblocks;
        const long long row = t * RV_GEMM_BM + r;
        const int col = kb * RV_GEMM_BK + ((ch ^ (r & 7)) << 3);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < N && col < K) v = *(const uint4*)(w + row * K + col);        // K is a multiple of 8
        out[i] = v;
    }
}

extern "C" long long rv_gemm_tiled_bytes(int N, int K) {
    const long long tiles = (N + RV_GEMM_BM - 1) / RV_GEMM_BM, kblocks = (K + RV_GEMM_BK - 1) / RV_GEMM_BK;
    return tiles * kblocks * RV_GEMM_BM * RV_GEMM_BK * 2;
}

extern "C" int rv_gemm_tile_weights(const void* w, void* out, int N, int K, void* stream) {
    if (N <= 0 || K <= 0 || K % 8 || ((uintptr_t)w | (uintptr_t)out) % 16)
        RV_FAIL("gemm_tile_weights: K = %d must be a multiple of 8 and the buffers 16-byte aligned", K);
    const int kblocks = (K + RV_GEMM_BK - 1) / RV_GEMM_BK;
    const long long chunks = rv_gemm_tiled_bytes(N, K) / 16;
    const int blocks = (int)((chunks + 255) / 256 < 148 * 32 ? (chunks + 255) / 256 : 148 * 32);
    tile_weights_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const bf16*)w, (uint4*)out, N, K,
                                                                   kblocks, chunks);
    RV_CHECK_LAUNCH("gemm_tile_weights");
    return 0;
}

// out[M, N] gets the normalised, rotated queries (its key and value columns are not written);
// keys and values go to `k_cache` / `v_cache` at `slot_mapping`.  Head size 64, bfloat16,
// M <= 16, N = (num_heads + 2 num_kv_heads) * 64.  Null weights: no norm; null tables: no
// rotation.
extern "C" int rv_gemm_tcgen05_qkv(const void* x, const void* w, void* out, int* status, int M,
                                   int N, int K, int num_heads, int num_kv_heads,
                                   const float* q_weight, const float* k_weight, float eps,
                                   const float* cos_table, const float* sin_table,
                                   const int* positions, const int* slot_mapping, void* k_cache,
                                   void* v_cache, const void* w_tiled, void* stream) {
    if (N != (num_heads + 2 * num_kv_heads) * 64)
        RV_FAIL("gemm_tcgen05_qkv: N = %d is not (heads + 2 kv heads) * 64", N);
    if (!slot_mapping || !k_cache || !v_cache || (cos_table && (!sin_table || !positions)))
        RV_FAIL("gemm_tcgen05_qkv: incomplete cache or rotation arguments");
    RvQkvEpilogue epi;
    epi.q_weight = q_weight;
    epi.k_weight = k_weight;
    epi.cos_table = cos_table;
    epi.sin_table = sin_table;
    epi.positions = positions;
    epi.slot_mapping = slot_mapping;
    epi.k_cache = (bf16*)k_cache;
    epi.v_cache = (bf16*)v_cache;
    epi.eps = eps;
    epi.num_heads = num_heads;
    epi.num_kv_heads = num_kv_heads;
    return gemm(x, w, out, RV_DTYPE_BF16, status, M, N, K, &epi, w_tiled, stream);
}
