// Sampling on the device: greedy argmax, and temperature with nucleus (top-p) filtering.
// One block per row of float32 logits, so only token ids cross to the host.
//
// argmax: the first maximum wins, NaN never wins, a row with nothing above -inf gives
// 0 (the reference's argmax.cu:1-4 and src/sampler.rs:68-78).
//
// sample: p_i = exp(l_i / T - max) (src/sampler.rs:80-91); the nucleus is the set
// {p_i >= tau} for the largest tau whose set has mass >= top_p * total, found by
// bisection on the bit pattern of tau (positive floats order like their bits); tokens
// tied with the last kept one are kept (the reference keeps a sorted prefix,
// src/sampler.rs:93-117).  The draw u in [0,1) is a counter-based hash of (seed,
// counter), so a request's stream depends on nothing else in the batch; the token is the
// first in index order whose cumulative kept mass reaches u * kept mass (the reference
// walks in descending-probability order with a stateful generator,
// src/sampler.rs:118-129).  Plain reference: tests/plain_ops.py sample_row.
#include "common.cuh"

// Stage 1: block (row, part) scans its slice of the row; stage 2 combines the parts.
// A candidate is (value, index); the better one has the larger value, or on a tie the
// smaller index, so the result does not depend on how the row is cut.
struct RvBest { float v; int i; };
__device__ __forceinline__ RvBest rv_better(RvBest a, RvBest b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ __forceinline__ RvBest rv_block_best(RvBest x, float* sv, int* si) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        RvBest y;
        y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
        x = rv_better(x, y);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = x.v; si[warp] = x.i; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        x.v = lane < nw ? sv[lane] : -INFINITY;
        x.i = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            RvBest y;
            y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
            y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
            x = rv_better(x, y);
        }
    }
    return x;   // valid in warp 0
}

__global__ void argmax_parts_kernel(const float* __restrict__ logits, float* __restrict__ part_v,
                                    int* __restrict__ part_i, int vocab, int parts) {
    rv_pdl_prologue();
    __shared__ float sv[32];
    __shared__ int si[32];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    const int per = (vocab + parts - 1) / parts;
    const int a = blockIdx.y * per, b = min(vocab, a + per);
    RvBest best = {-INFINITY, 0x7fffffff};
    // four loads in flight per thread (a load and its compare per iteration would cost one
    // memory latency each); compared in index order, and strict, so the earliest maximum stays
    const int bd = blockDim.x;
    for (int i = a + threadIdx.x; i < b; i += 4 * bd) {
        float v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = i + k * bd < b ? row[i + k * bd] : -INFINITY;
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (v[k] > best.v) { best.v = v[k]; best.i = i + k * bd; }   // false for NaN
    }
    best = rv_block_best(best, sv, si);
    if (threadIdx.x == 0) {
        part_v[blockIdx.x * parts + blockIdx.y] = best.v;
        part_i[blockIdx.x * parts + blockIdx.y] = best.i;
    }
}

__global__ void argmax_final_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i,
                                    int* __restrict__ out, int parts) {
    rv_pdl_prologue();
    RvBest best = {-INFINITY, 0x7fffffff};
    for (int p = threadIdx.x; p < parts; p += 32) {
        RvBest c = {part_v[blockIdx.x * parts + p], part_i[blockIdx.x * parts + p]};
        best = rv_better(best, c);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        RvBest y;
        y.v = __shfl_xor_sync(0xffffffffu, best.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, best.i, o);
        best = rv_better(best, y);
    }
    if (threadIdx.x == 0) out[blockIdx.x] = best.i == 0x7fffffff ? 0 : best.i;
}

#define RV_ARGMAX_MAX_PARTS 64

// `scratch` holds rows * parts (value, index) pairs: rows * parts * 8 bytes, parts as
// given by rv_argmax_parts.
extern "C" int rv_argmax_parts(int n_rows, int vocab) {
    int parts = 1;
    const int want = 2 * rv_sm_count();        // two blocks per SM
    while (parts < RV_ARGMAX_MAX_PARTS && n_rows * parts < want && vocab / (parts * 2) >= 1024) parts *= 2;
    return parts;
}

extern "C" int rv_argmax(const float* logits, int* out, void* scratch, long long scratch_bytes,
                         int n_rows, int vocab, void* stream) {
    if (n_rows == 0) return 0;
    if (n_rows < 0 || vocab <= 0) RV_FAIL("argmax: bad sizes");
    if (n_rows > 65535) RV_FAIL("argmax: too many rows for one launch");
    const int parts = rv_argmax_parts(n_rows, vocab);
    if ((long long)n_rows * parts * 8 > scratch_bytes) RV_FAIL("argmax: scratch too small");
    float* part_v = (float*)scratch;
    int* part_i = (int*)((char*)scratch + (size_t)n_rows * parts * 4);
    cudaStream_t s = (cudaStream_t)stream;
    rv_launch(argmax_parts_kernel, dim3(dim3(n_rows, parts)), dim3(256), 0, s, logits, part_v, part_i, vocab, parts);
    RV_CHECK_LAUNCH("argmax");
    rv_launch(argmax_final_kernel, dim3(n_rows), dim3(32), 0, s, part_v, part_i, out, parts);
    RV_CHECK_LAUNCH("argmax");
    return 0;
}

__device__ __forceinline__ float rv_uniform(unsigned long long seed, unsigned long long counter) {
    unsigned long long z = seed + (counter + 1ull) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

#define RV_SAMPLE_THREADS 1024

__global__ void __launch_bounds__(RV_SAMPLE_THREADS) sample_kernel(
    const float* __restrict__ logits, const float* __restrict__ temperature,
    const float* __restrict__ top_p, const long long* __restrict__ seed,
    const long long* __restrict__ counter, int* __restrict__ out, int vocab) {
    rv_pdl_prologue();
    __shared__ float scratch[33];
    __shared__ float seg_sum[RV_SAMPLE_THREADS];
    __shared__ int chosen_thread;
    const int m = blockIdx.x;
    const float* row = logits + (size_t)m * vocab;
    const float T = temperature[m];
    const float inv_t = 1.f / T;
    // each thread owns a contiguous segment of the vocabulary
    const int seg = (vocab + blockDim.x - 1) / blockDim.x;
    const int a = min(vocab, (int)threadIdx.x * seg), b = min(vocab, a + seg);

    float mx = -INFINITY;
    for (int i = a; i < b; ++i) mx = fmaxf(mx, row[i] * inv_t);
    mx = rv_block_max(mx, scratch);
    float sum = 0.f;
    for (int i = a; i < b; ++i) sum += expf(row[i] * inv_t - mx);
    const float total = rv_block_sum(sum, scratch);

    // nucleus threshold: the largest tau with mass{p >= tau} >= top_p * total
    float tau = 0.f;
    const float tp = top_p[m];
    if (tp < 1.f) {
        const float need = tp * total;
        unsigned lo = 0u, hi = 0x3f800000u;   // p is in (0, 1]; tau = lo always qualifies
        while (lo < hi) {
            const unsigned mid = lo + (hi - lo + 1) / 2;
            const float cand = __uint_as_float(mid);
            float mass = 0.f;
            for (int i = a; i < b; ++i) {
                const float p = expf(row[i] * inv_t - mx);
                if (p >= cand) mass += p;
            }
            mass = rv_block_sum(mass, scratch);
            if (mass >= need) lo = mid; else hi = mid - 1;
        }
        tau = __uint_as_float(lo);
    }
    float kept = 0.f;
    for (int i = a; i < b; ++i) {
        const float p = expf(row[i] * inv_t - mx);
        if (p >= tau) kept += p;
    }
    seg_sum[threadIdx.x] = kept;
    const float kept_total = rv_block_sum(kept, scratch);   // also orders the seg_sum writes
    const float target = rv_uniform((unsigned long long)seed[m], (unsigned long long)counter[m]) *
                         kept_total;
    if (threadIdx.x == 0) {
        // walk the segment sums in order; 1024 additions
        float acc = 0.f;
        int t = 0, last = 0;
        for (t = 0; t < (int)blockDim.x; ++t) {
            if (seg_sum[t] > 0.f) last = t;
            if (seg_sum[t] > 0.f && acc + seg_sum[t] >= target) break;
            acc += seg_sum[t];
        }
        if (t == (int)blockDim.x) {   // rounding left the target past the end
            t = last;
            acc = -INFINITY;
        }
        chosen_thread = t;
        scratch[0] = acc;
    }
    __syncthreads();
    if ((int)threadIdx.x == chosen_thread) {
        float acc = scratch[0];
        int pick = -1, last = a;
        for (int i = a; i < b; ++i) {
            const float p = expf(row[i] * inv_t - mx);
            if (p >= tau && p > 0.f) {
                last = i;
                acc += p;
                if (acc >= target) {
                    pick = i;
                    break;
                }
            }
        }
        out[m] = pick >= 0 ? pick : last;
    }
}

extern "C" int rv_sample(const float* logits, const float* temperature, const float* top_p,
                         const long long* seed, const long long* counter, int* out, int n_rows,
                         int vocab, void* stream) {
    if (n_rows == 0) return 0;
    if (n_rows < 0 || vocab <= 0) RV_FAIL("sample: bad sizes");
    rv_launch(sample_kernel, dim3(n_rows), dim3(RV_SAMPLE_THREADS), 0, (cudaStream_t)stream, 
        logits, temperature, top_p, seed, counter, out, vocab);
    RV_CHECK_LAUNCH("sample");
    return 0;
}
