// Sampling on the device: greedy argmax, and temperature with nucleus (top-p) filtering.
// One block per row of float32 logits, so only token ids cross to the host.
//
// argmax: the first maximum wins, NaN never wins, a row with nothing above -inf gives
// 0 (the reference's argmax.cu:1-4 and src/sampler.rs:68-78).
//
// sample: a row with T <= 0 is greedy (as argmax).  Otherwise p_i = exp(l_i / T - max)
// (src/sampler.rs:80-91); the nucleus is the set
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

// A row whose temperature is not positive is greedy: the first maximum, NaN never wins, nothing
// above -inf gives 0 (as `rv_argmax`).  Every thread of the block calls it.
__device__ __forceinline__ void rv_sample_greedy_row(const float* row, int a, int b, int* out) {
    __shared__ float gv[32];
    __shared__ int gi[32];
    RvBest best = {-INFINITY, 0x7fffffff};
    for (int i = a; i < b; ++i) {
        const float v = row[i];
        if (v > best.v) best = RvBest{v, i};
    }
    best = rv_block_best(best, gv, gi);
    if (threadIdx.x == 0) *out = best.i == 0x7fffffff ? 0 : best.i;
}

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
    if (!(T > 0.f)) {
        rv_sample_greedy_row(row, a, b, out + m);
        return;
    }

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

// The same with the row kept on the chip and read from memory once, coalesced.  Warp w owns
// the `rows * 32` consecutive values from w * rows * 32 on, lane l the values j * 32 + l of
// them: a load of the warp is 128 contiguous bytes.  A thread keeps its first RV_SAMPLE_REGS
// values in registers and the rest in shared memory (value j of thread t at [j][t]: no bank
// conflicts).  The maximum, the sum and the thirty-odd passes of the bisection run on chip.
// The walk to the drawn token follows index order: per warp the kept mass row of 32 by row of 32
// (each row summed over the lanes by the same shuffle tree), the warps' totals in order to find
// the warp, the rows again to find the row, a prefix over the lanes to find the token: 32 + rows
// + 5 steps instead of 1024 + values per thread.  The sums are taken in another order than in
// `sample_kernel`, so a draw that falls within float32 rounding of a boundary may pick the
// neighbouring kept token there; both follow the definition in tests/plain_ops.py sample_row.
// Rows of up to 1024 * (RV_SAMPLE_REGS + RV_SAMPLE_SMEM) values.
#define RV_SAMPLE_REGS 20
#define RV_SAMPLE_SMEM 52

#define RV_FOR_EACH_P(BODY)                                                     \
    do {                                                                        \
        _Pragma("unroll") for (int i_ = 0; i_ < RV_SAMPLE_REGS; ++i_) {         \
            if (i_ < rows) { float& p = pr[i_]; BODY; }                         \
        }                                                                       \
        for (int i_ = RV_SAMPLE_REGS; i_ < rows; ++i_) {                        \
            float& p = ps[(i_ - RV_SAMPLE_REGS) * RV_SAMPLE_THREADS + threadIdx.x]; \
            BODY;                                                               \
        }                                                                       \
    } while (0)

__global__ void __launch_bounds__(RV_SAMPLE_THREADS) sample_onchip_kernel(
    const float* __restrict__ logits, const float* __restrict__ temperature,
    const float* __restrict__ top_p, const long long* __restrict__ seed,
    const long long* __restrict__ counter, int* __restrict__ out, int vocab, int rows) {
    rv_pdl_prologue();
    extern __shared__ float ps[];
    __shared__ float scratch[33];
    __shared__ float warp_total[32];
    const int m = blockIdx.x;
    const float* row = logits + (size_t)m * vocab;
    const float T = temperature[m];
    const float inv_t = 1.f / T;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int base = warp * rows * 32 + lane;            // this thread's value j is row[base + 32 j]
    if (!(T > 0.f)) {
        // greedy: this layout would do as well, but one definition of "first maximum" is enough
        const int seg = (vocab + blockDim.x - 1) / blockDim.x;
        const int a = min(vocab, (int)threadIdx.x * seg);
        rv_sample_greedy_row(row, a, min(vocab, a + seg), out + m);
        return;
    }
    float pr[RV_SAMPLE_REGS];

    // the only pass over global memory; values past the row's end count as -inf (probability 0)
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < RV_SAMPLE_REGS; ++i)
        pr[i] = (i < rows && base + 32 * i < vocab) ? row[base + 32 * i] * inv_t : -INFINITY;
#pragma unroll
    for (int i = 0; i < RV_SAMPLE_REGS; ++i) mx = fmaxf(mx, pr[i]);
    for (int i0 = RV_SAMPLE_REGS; i0 < rows; i0 += 8) {
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k)
            v[k] = (i0 + k < rows && base + 32 * (i0 + k) < vocab) ? row[base + 32 * (i0 + k)] * inv_t
                                                                  : -INFINITY;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (i0 + k < rows) ps[(i0 + k - RV_SAMPLE_REGS) * RV_SAMPLE_THREADS + threadIdx.x] = v[k];
            mx = fmaxf(mx, v[k]);
        }
    }
    mx = rv_block_max(mx, scratch);
    float sum = 0.f;
    RV_FOR_EACH_P(p = expf(p - mx); sum += p);
    const float total = rv_block_sum(sum, scratch);

    float tau = 0.f;
    const float tp = top_p[m];
    if (tp < 1.f) {
        const float need = tp * total;
        unsigned lo = 0u, hi = 0x3f800000u;   // p is in (0, 1]; tau = lo always qualifies
        while (lo < hi) {
            const unsigned mid = lo + (hi - lo + 1) / 2;
            const float cand = __uint_as_float(mid);
            float mass = 0.f;
            RV_FOR_EACH_P(if (p >= cand) mass += p);
            mass = rv_block_sum(mass, scratch);
            if (mass >= need) lo = mid; else hi = mid - 1;
        }
        tau = __uint_as_float(lo);
    }
    // the kept mass of this warp's values, row of 32 by row of 32 in index order
    float acc = 0.f;
    RV_FOR_EACH_P(acc += rv_warp_sum((p >= tau && p > 0.f) ? p : 0.f));
    if (lane == 0) warp_total[warp] = acc;
    __syncthreads();
    float kept_total = 0.f;
    for (int w = 0; w < 32; ++w) kept_total += warp_total[w];
    const float target = rv_uniform((unsigned long long)seed[m], (unsigned long long)counter[m]) *
                         kept_total;
    // the warp in which the cumulative kept mass reaches the target (every thread finds the same)
    float before = 0.f;
    int chosen = -1, last_warp = 0;
    for (int w = 0; w < 32; ++w) {
        const float t = warp_total[w];
        if (t > 0.f) {
            last_warp = w;
            if (chosen < 0 && before + t >= target) chosen = w;
        }
        if (chosen < 0) before += t;
    }
    bool past_end = false;
    if (chosen < 0) {                 // rounding left the target past the end: the last kept token
        chosen = last_warp;
        past_end = true;
    }
    if (warp != chosen) return;
    float run = before;
    int pick = -1, last = -1;
    RV_FOR_EACH_P(
        {
            const float q = (p >= tau && p > 0.f) ? p : 0.f;
            const float rowsum = rv_warp_sum(q);
            const unsigned keepers = __ballot_sync(0xffffffffu, q > 0.f);
            if (keepers) last = warp * rows * 32 + i_ * 32 + (31 - __clz((int)keepers));
            if (pick < 0 && !past_end && rowsum > 0.f && run + rowsum >= target) {
                // inclusive prefix over the lanes, then the first kept lane that reaches the target
                float pre = q;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const float up = __shfl_up_sync(0xffffffffu, pre, o);
                    if (lane >= o) pre += up;
                }
                const unsigned hit = __ballot_sync(0xffffffffu, q > 0.f && run + pre >= target);
                const unsigned take = hit ? hit : keepers;          // rounding: the row's last keeper
                const int l = hit ? __ffs((int)take) - 1 : 31 - __clz((int)take);
                pick = warp * rows * 32 + i_ * 32 + l;
            }
            run += rowsum;
        });
    if (lane == 0) out[m] = pick >= 0 ? pick : (last >= 0 ? last : 0);
}

// 1: rows that fit stay on the chip (the default); 0: every pass re-reads the logits
// (RVLLM_SAMPLE_ONCHIP=0).  The switch is for tests and timing.
static int rv_sample_onchip = -1;
extern "C" void rv_sample_set_onchip(int on) { rv_sample_onchip = on ? 1 : 0; }

extern "C" int rv_sample(const float* logits, const float* temperature, const float* top_p,
                         const long long* seed, const long long* counter, int* out, int n_rows,
                         int vocab, void* stream) {
    if (n_rows == 0) return 0;
    if (n_rows < 0 || vocab <= 0) RV_FAIL("sample: bad sizes");
    // rows of 32 values per warp: 32 warps cover the row
    const int rows = (vocab + 1023) / 1024;
    if (rv_sample_onchip < 0) {
        const char* e = getenv("RVLLM_SAMPLE_ONCHIP");
        rv_sample_onchip = (e && e[0] == '0') ? 0 : 1;
    }
    if (rv_sample_onchip && rows <= RV_SAMPLE_REGS + RV_SAMPLE_SMEM) {
        // the row stays on the chip: registers, and shared memory for what exceeds them
        const size_t smem = rows > RV_SAMPLE_REGS
            ? (size_t)(rows - RV_SAMPLE_REGS) * RV_SAMPLE_THREADS * sizeof(float) : 0;
        static size_t raised = 0;
        if (smem > 48 * 1024 && smem > raised) {
            cudaError_t e = cudaFuncSetAttribute(sample_onchip_kernel,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) RV_FAIL("sample: %s", cudaGetErrorString(e));
            raised = smem;
        }
        rv_launch(sample_onchip_kernel, dim3(n_rows), dim3(RV_SAMPLE_THREADS), smem,
                  (cudaStream_t)stream, logits, temperature, top_p, seed, counter, out, vocab, rows);
    } else {
        rv_launch(sample_kernel, dim3(n_rows), dim3(RV_SAMPLE_THREADS), 0, (cudaStream_t)stream,
                  logits, temperature, top_p, seed, counter, out, vocab);
    }
    RV_CHECK_LAUNCH("sample");
    return 0;
}
