// Gated short convolution for any mixture of prompt portions and single tokens:
// gate B*x, load of the request's state, the causal taps, gate C, and the store of the
// new state, in one kernel.
//
//   proj[t] = (B | C | x), three chunks of `hidden` channels (plus the optional bias)
//   bx[t]   = B[t] * x[t]
//   window  = the request's taps-1 previous bx rows (the state; zeros before position
//             0), then this step's bx rows
//   out[t]  = C[t] * (sum_k filter[c, k] * window[t + k] + conv_bias[c])
//   state'  = the window's last taps-1 rows
//
// One thread owns one channel of one chunk of 32 consecutive tokens of one request and
// slides the window through registers.  The thread of chunk 0 is the only one that
// reads or writes the state of its (request, channel): it reads the old rows before
// anything else and writes the new rows last, so no other thread can see a half-updated
// state.  Later chunks rebuild their first taps-1 window rows from proj.  The state is
// float32 whatever the storage type, so a bx value is the same number whether it comes
// from the state or is recomputed from proj.
//
// Reference counterparts: short_conv_bx and short_conv_filter_gate (short_conv.cu) with
// per-item device-to-device copies around them (src/cuda/model.rs:599-677,
// src/cuda/conv_cache.rs:61-115).  Plain reference: tests/plain_ops.py short_conv.
#include "common.cuh"

#define RV_CONV_MAX_TAPS 8
#define RV_CONV_CHUNK 32

template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ proj, const float* __restrict__ filter,
                                  const float* __restrict__ in_bias,
                                  const float* __restrict__ conv_bias, float* __restrict__ state,
                                  const int* __restrict__ q_start, const int* __restrict__ state_slot,
                                  const int* __restrict__ start_pos, T* __restrict__ out,
                                  int hidden, int taps) {
    rv_pdl_prologue();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= hidden) return;
    const int r = blockIdx.y;
    const int q0 = q_start[r];
    const int qlen = q_start[r + 1] - q0;
    const int t0 = blockIdx.z * RV_CONV_CHUNK;
    if (t0 >= qlen) return;
    const int slot = state_slot[r];
    const int hist = taps - 1;
    const bool has_state = slot >= 0 && start_pos[r] > 0 && hist > 0;
    float* st = slot >= 0 ? state + (size_t)slot * hist * hidden + c : nullptr;

    float f[RV_CONV_MAX_TAPS];
#pragma unroll
    for (int k = 0; k < RV_CONV_MAX_TAPS; ++k) f[k] = k < taps ? filter[(size_t)c * taps + k] : 0.f;
    const float bb = in_bias ? in_bias[c] : 0.f;
    const float bc = in_bias ? in_bias[hidden + c] : 0.f;
    const float bxb = in_bias ? in_bias[2 * hidden + c] : 0.f;
    const float cb = conv_bias ? conv_bias[c] : 0.f;
    const size_t stride = (size_t)3 * hidden;

    auto bx_at = [&](int rel) -> float {   // B*x of the request's rel-th token of this step
        const T* p = proj + (size_t)(q0 + rel) * stride + c;
        return (rv_load(p) + bb) * (rv_load(p + 2 * hidden) + bxb);
    };

    // window rows before token t0; in chunk 0 they are the old state
    float old[RV_CONV_MAX_TAPS - 1];
    float win[RV_CONV_MAX_TAPS - 1];
#pragma unroll
    for (int i = 0; i < RV_CONV_MAX_TAPS - 1; ++i) {
        old[i] = 0.f;
        win[i] = 0.f;
        if (i < hist) {
            const int rel = t0 - hist + i;
            if (rel >= 0) {
                win[i] = bx_at(rel);
            } else if (has_state) {
                old[i] = st[(size_t)(hist + rel) * hidden];
                win[i] = old[i];
            }
        }
    }
    const int t1 = min(t0 + RV_CONV_CHUNK, qlen);
    for (int t = t0; t < t1; ++t) {
        const T* p = proj + (size_t)(q0 + t) * stride + c;
        const float bx = (rv_load(p) + bb) * (rv_load(p + 2 * hidden) + bxb);
        const float gate_c = rv_load(p + hidden) + bc;
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < RV_CONV_MAX_TAPS - 1; ++k)
            if (k < hist) acc += f[k] * win[k];
        acc += f[hist] * bx;
        rv_store(out + (size_t)(q0 + t) * hidden + c, gate_c * (acc + cb));
#pragma unroll
        for (int k = 0; k < RV_CONV_MAX_TAPS - 2; ++k)
            if (k + 1 < hist) win[k] = win[k + 1];
        if (hist > 0) {
#pragma unroll
            for (int k = 0; k < RV_CONV_MAX_TAPS - 1; ++k)
                if (k == hist - 1) win[k] = bx;
        }
    }
    if (t0 == 0 && st && hist > 0) {
        // new state row i = window row qlen + i; window row w < hist is old[w]
#pragma unroll
        for (int i = 0; i < RV_CONV_MAX_TAPS - 1; ++i) {
            if (i < hist) {
                const int w = qlen + i;
                float v = 0.f;
                if (w >= hist) {
                    v = bx_at(w - hist);
                } else {
#pragma unroll
                    for (int k = 0; k < RV_CONV_MAX_TAPS - 1; ++k)
                        if (k == w) v = old[k];
                }
                st[(size_t)i * hidden] = v;
            }
        }
    }
}

// The same for filters of at most 4 taps and widths that are a multiple of 4: a thread owns
// four adjacent channels and moves them with one 8-byte (bfloat16) or 16-byte (float32)
// access per row, which is what makes long prompt portions run at memory speed.
__device__ __forceinline__ float4 rv_conv_load4(const float* p) { return *(const float4*)p; }
__device__ __forceinline__ float4 rv_conv_load4(const __nv_bfloat16* p) {
    const uint2 raw = *(const uint2*)p;
    const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&raw.x);
    const float2 b = __bfloat1622float2(*(const __nv_bfloat162*)&raw.y);
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void rv_conv_store4(float* p, float4 v) { *(float4*)p = v; }
__device__ __forceinline__ void rv_conv_store4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *(const unsigned*)&a;
    raw.y = *(const unsigned*)&b;
    *(uint2*)p = raw;
}
__device__ __forceinline__ float4 rv_f4_add(float4 a, float4 b) {
    return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}
__device__ __forceinline__ float4 rv_f4_mul(float4 a, float4 b) {
    return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w);
}

#define RV_CONV_VEC_TAPS 4

template <typename T>
__global__ void short_conv_vec4_kernel(const T* __restrict__ proj, const float* __restrict__ filter,
                                       const float* __restrict__ in_bias,
                                       const float* __restrict__ conv_bias, float* __restrict__ state,
                                       const int* __restrict__ q_start,
                                       const int* __restrict__ state_slot,
                                       const int* __restrict__ start_pos, T* __restrict__ out,
                                       int hidden, int taps) {
    // index arrays, filter and biases do not depend on the previous kernel: they are requested
    // before the wait for it
    rv_pdl_launch_dependents();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (c >= hidden) return;
    const int r = blockIdx.y;
    const int q0 = q_start[r];
    const int qlen = q_start[r + 1] - q0;
    const int t0 = blockIdx.z * RV_CONV_CHUNK;
    if (t0 >= qlen) return;
    const int slot = state_slot[r];
    const int hist = taps - 1;
    const bool has_state = slot >= 0 && start_pos[r] > 0 && hist > 0;
    float* st = slot >= 0 ? state + (size_t)slot * hist * hidden + c : nullptr;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);

    float4 f[RV_CONV_VEC_TAPS];                        // f[k] = tap k of the four channels
#pragma unroll
    for (int k = 0; k < RV_CONV_VEC_TAPS; ++k)
        f[k] = k < taps ? make_float4(filter[(size_t)c * taps + k], filter[(size_t)(c + 1) * taps + k],
                                      filter[(size_t)(c + 2) * taps + k],
                                      filter[(size_t)(c + 3) * taps + k]) : zero;
    const float4 bb = in_bias ? *(const float4*)(in_bias + c) : zero;
    const float4 bc = in_bias ? *(const float4*)(in_bias + hidden + c) : zero;
    const float4 bxb = in_bias ? *(const float4*)(in_bias + 2 * hidden + c) : zero;
    const float4 cb = conv_bias ? *(const float4*)(conv_bias + c) : zero;
    const size_t stride = (size_t)3 * hidden;

    auto bx_at = [&](int rel) -> float4 {
        const T* p = proj + (size_t)(q0 + rel) * stride + c;
        return rv_f4_mul(rv_f4_add(rv_conv_load4(p), bb), rv_f4_add(rv_conv_load4(p + 2 * hidden), bxb));
    };
    rv_pdl_wait();
    float4 old[RV_CONV_VEC_TAPS - 1], win[RV_CONV_VEC_TAPS - 1];
#pragma unroll
    for (int i = 0; i < RV_CONV_VEC_TAPS - 1; ++i) {
        old[i] = zero;
        win[i] = zero;
        if (i < hist) {
            const int rel = t0 - hist + i;
            if (rel >= 0) {
                win[i] = bx_at(rel);
            } else if (has_state) {
                old[i] = *(const float4*)(st + (size_t)(hist + rel) * hidden);
                win[i] = old[i];
            }
        }
    }
    const int t1 = min(t0 + RV_CONV_CHUNK, qlen);
    for (int t = t0; t < t1; ++t) {
        const T* p = proj + (size_t)(q0 + t) * stride + c;
        const float4 bx = rv_f4_mul(rv_f4_add(rv_conv_load4(p), bb),
                                    rv_f4_add(rv_conv_load4(p + 2 * hidden), bxb));
        const float4 gate_c = rv_f4_add(rv_conv_load4(p + hidden), bc);
        float4 acc = zero;
#pragma unroll
        for (int k = 0; k < RV_CONV_VEC_TAPS - 1; ++k)
            if (k < hist) acc = rv_f4_add(acc, rv_f4_mul(f[k], win[k]));
#pragma unroll
        for (int k = 0; k < RV_CONV_VEC_TAPS; ++k)
            if (k == hist) acc = rv_f4_add(acc, rv_f4_mul(f[k], bx));
        rv_conv_store4(out + (size_t)(q0 + t) * hidden + c, rv_f4_mul(gate_c, rv_f4_add(acc, cb)));
#pragma unroll
        for (int k = 0; k < RV_CONV_VEC_TAPS - 2; ++k)
            if (k + 1 < hist) win[k] = win[k + 1];
#pragma unroll
        for (int k = 0; k < RV_CONV_VEC_TAPS - 1; ++k)
            if (k == hist - 1) win[k] = bx;
    }
    if (t0 == 0 && st && hist > 0 && qlen <= RV_CONV_CHUNK) {
        // the whole portion went through this thread: the window it ends with is the new state
        // (nothing is read again, so a single token's step has one dependent load fewer)
#pragma unroll
        for (int i = 0; i < RV_CONV_VEC_TAPS - 1; ++i)
            if (i < hist) *(float4*)(st + (size_t)i * hidden) = win[i];
    } else if (t0 == 0 && st && hist > 0) {
#pragma unroll
        for (int i = 0; i < RV_CONV_VEC_TAPS - 1; ++i) {
            if (i < hist) {
                const int w = qlen + i;
                float4 v = zero;
                if (w >= hist) {
                    v = bx_at(w - hist);
                } else {
#pragma unroll
                    for (int k = 0; k < RV_CONV_VEC_TAPS - 1; ++k)
                        if (k == w) v = old[k];
                }
                *(float4*)(st + (size_t)i * hidden) = v;
            }
        }
    }
}

// Long prompt portions: a thread owns eight adjacent channels (one 16-byte access per bfloat16
// row) of a chunk of 16 tokens and requests the rows of half a chunk (B, C and x of 8 tokens:
// 24 independent loads; a quarter chunk in float32) before it uses any of them, so that enough bytes are in flight to
// run at memory speed; the sums are formed in the same order as in the kernels above, so the
// three give the same numbers.  Filters of at most 4 taps, widths that are a multiple of 8.
#define RV_CONV_WIDE_CHUNK 16

struct RvRaw8Bf16 { uint4 v; };
struct RvRaw8F32 { float4 a, b; };
template <typename T> struct RvRaw8;
template <> struct RvRaw8<__nv_bfloat16> { typedef RvRaw8Bf16 type; };
template <> struct RvRaw8<float> { typedef RvRaw8F32 type; };
__device__ __forceinline__ RvRaw8Bf16 rv_conv_raw8(const __nv_bfloat16* p) {
    RvRaw8Bf16 r;
    r.v = *(const uint4*)p;
    return r;
}
__device__ __forceinline__ RvRaw8F32 rv_conv_raw8(const float* p) {
    RvRaw8F32 r;
    r.a = *(const float4*)p;
    r.b = *(const float4*)(p + 4);
    return r;
}
__device__ __forceinline__ void rv_conv_unpack8(const RvRaw8Bf16& r, float (&o)[8]) {
    // a bfloat16 is the upper half of the float32 of the same value
    o[0] = __uint_as_float(r.v.x << 16); o[1] = __uint_as_float(r.v.x & 0xffff0000u);
    o[2] = __uint_as_float(r.v.y << 16); o[3] = __uint_as_float(r.v.y & 0xffff0000u);
    o[4] = __uint_as_float(r.v.z << 16); o[5] = __uint_as_float(r.v.z & 0xffff0000u);
    o[6] = __uint_as_float(r.v.w << 16); o[7] = __uint_as_float(r.v.w & 0xffff0000u);
}
__device__ __forceinline__ void rv_conv_unpack8(const RvRaw8F32& r, float (&o)[8]) {
    o[0] = r.a.x; o[1] = r.a.y; o[2] = r.a.z; o[3] = r.a.w;
    o[4] = r.b.x; o[5] = r.b.y; o[6] = r.b.z; o[7] = r.b.w;
}
__device__ __forceinline__ void rv_conv_store8(__nv_bfloat16* p, const float (&v)[8]) {
    union { __nv_bfloat162 h; unsigned u; } a, b, c, d;
    a.h = __floats2bfloat162_rn(v[0], v[1]);
    b.h = __floats2bfloat162_rn(v[2], v[3]);
    c.h = __floats2bfloat162_rn(v[4], v[5]);
    d.h = __floats2bfloat162_rn(v[6], v[7]);
    *(uint4*)p = make_uint4(a.u, b.u, c.u, d.u);
}
__device__ __forceinline__ void rv_conv_store8(float* p, const float (&v)[8]) {
    *(float4*)p = make_float4(v[0], v[1], v[2], v[3]);
    *(float4*)(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

template <typename T, int TAPS>
__global__ void __launch_bounds__(128) short_conv_wide_kernel(
    const T* __restrict__ proj, const float* __restrict__ filter, const float* __restrict__ in_bias,
    const float* __restrict__ conv_bias, float* __restrict__ state, const int* __restrict__ q_start,
    const int* __restrict__ state_slot, const int* __restrict__ start_pos, T* __restrict__ out,
    int hidden) {
    typedef typename RvRaw8<T>::type Raw;
    constexpr int ROWS = sizeof(T) == 2 ? 8 : 4;       // rows requested together: 24 loads of 16 bytes
    constexpr int HIST = TAPS - 1;
    rv_pdl_launch_dependents();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= hidden) return;
    const int r = blockIdx.y;
    const int q0 = q_start[r];
    const int qlen = q_start[r + 1] - q0;
    const int t0 = blockIdx.z * RV_CONV_WIDE_CHUNK;
    if (t0 >= qlen) return;
    const int slot = state_slot[r];
    const bool has_state = slot >= 0 && start_pos[r] > 0 && HIST > 0;
    float* st = slot >= 0 ? state + (size_t)slot * HIST * hidden + c : nullptr;

    // the eight channels' filters lie side by side: 8 * TAPS floats from a 16-byte boundary
    float flat[8 * TAPS];
#pragma unroll
    for (int j = 0; j < 2 * TAPS; ++j) {
        const float4 v = *(const float4*)(filter + (size_t)c * TAPS + 4 * j);
        flat[4 * j] = v.x; flat[4 * j + 1] = v.y; flat[4 * j + 2] = v.z; flat[4 * j + 3] = v.w;
    }
    float bb[8], bc[8], bxb[8], cb[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        bb[i] = in_bias ? in_bias[c + i] : 0.f;
        bc[i] = in_bias ? in_bias[hidden + c + i] : 0.f;
        bxb[i] = in_bias ? in_bias[2 * hidden + c + i] : 0.f;
        cb[i] = conv_bias ? conv_bias[c + i] : 0.f;
    }
    const size_t stride = (size_t)3 * hidden;
    auto bx_of = [&](const Raw& rb, const Raw& rx, float (&o)[8]) {
        float b[8], x[8];
        rv_conv_unpack8(rb, b);
        rv_conv_unpack8(rx, x);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = (b[i] + bb[i]) * (x[i] + bxb[i]);
    };
    auto bx_at = [&](int rel, float (&o)[8]) {
        const T* p = proj + (size_t)(q0 + rel) * stride + c;
        bx_of(rv_conv_raw8(p), rv_conv_raw8(p + 2 * hidden), o);
    };
    rv_pdl_wait();
    float old[HIST > 0 ? HIST : 1][8], win[HIST > 0 ? HIST : 1][8];
#pragma unroll
    for (int k = 0; k < HIST; ++k) {
#pragma unroll
        for (int i = 0; i < 8; ++i) old[k][i] = win[k][i] = 0.f;
        const int rel = t0 - HIST + k;
        if (rel >= 0) {
            bx_at(rel, win[k]);
        } else if (has_state) {
            const float* sp = st + (size_t)(HIST + rel) * hidden;
            const float4 a = *(const float4*)sp, b = *(const float4*)(sp + 4);
            old[k][0] = a.x; old[k][1] = a.y; old[k][2] = a.z; old[k][3] = a.w;
            old[k][4] = b.x; old[k][5] = b.y; old[k][6] = b.z; old[k][7] = b.w;
#pragma unroll
            for (int i = 0; i < 8; ++i) win[k][i] = old[k][i];
        }
    }
    const int t1 = min(t0 + RV_CONV_WIDE_CHUNK, qlen);
    for (int tb = t0; tb < t1; tb += ROWS) {
        // every row of this part of the chunk is requested before the first is used (a row past
        // the portion's end reads the last valid row again and is not used)
        Raw rb[ROWS], rc[ROWS], rx[ROWS];
#pragma unroll
        for (int j = 0; j < ROWS; ++j) {
            const T* p = proj + (size_t)(q0 + min(tb + j, t1 - 1)) * stride + c;
            rb[j] = rv_conv_raw8(p);
            rc[j] = rv_conv_raw8(p + hidden);
            rx[j] = rv_conv_raw8(p + 2 * hidden);
        }
#pragma unroll
        for (int j = 0; j < ROWS; ++j) {
            if (tb + j < t1) {
                float bx[8], gate_c[8], res[8];
                bx_of(rb[j], rx[j], bx);
                rv_conv_unpack8(rc[j], gate_c);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float acc = 0.f;
#pragma unroll
                    for (int k = 0; k < HIST; ++k) acc += flat[i * TAPS + k] * win[k][i];
                    acc += flat[i * TAPS + HIST] * bx[i];
                    res[i] = (gate_c[i] + bc[i]) * (acc + cb[i]);
                }
                rv_conv_store8(out + (size_t)(q0 + tb + j) * hidden + c, res);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
#pragma unroll
                    for (int k = 0; k + 1 < HIST; ++k) win[k][i] = win[k + 1][i];
                    if (HIST > 0) win[HIST > 0 ? HIST - 1 : 0][i] = bx[i];
                }
            }
        }
    }
    if (t0 == 0 && st && HIST > 0) {
#pragma unroll
        for (int k = 0; k < HIST; ++k) {
            const int w = qlen + k;                    // window row of the new state's row k
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.f;
            if (w >= HIST) {
                bx_at(w - HIST, v);
            } else {
#pragma unroll
                for (int kk = 0; kk < HIST; ++kk)
                    if (kk == w) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) v[i] = old[kk][i];
                    }
            }
            float* sp = st + (size_t)k * hidden;
            *(float4*)sp = make_float4(v[0], v[1], v[2], v[3]);
            *(float4*)(sp + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
    }
}

template <typename T>
static void short_conv_wide_launch(dim3 grid, cudaStream_t stream, const void* proj, const float* filter,
                                   const float* in_bias, const float* conv_bias, float* state,
                                   const int* q_start, const int* state_slot, const int* start_pos,
                                   void* out, int hidden, int taps) {
#define RV_CONV_WIDE_CASE(N)                                                                     \
    case N:                                                                                      \
        rv_launch(short_conv_wide_kernel<T, N>, grid, dim3(128), 0, stream, (const T*)proj, filter, \
                  in_bias, conv_bias, state, q_start, state_slot, start_pos, (T*)out, hidden);   \
        break;
    switch (taps) {
        RV_CONV_WIDE_CASE(1)
        RV_CONV_WIDE_CASE(2)
        RV_CONV_WIDE_CASE(3)
        RV_CONV_WIDE_CASE(4)
    }
#undef RV_CONV_WIDE_CASE
}

extern "C" int rv_short_conv(const void* proj, int dtype, const float* filter, const float* in_bias,
                             const float* conv_bias, float* state, const int* q_start,
                             const int* state_slot, const int* start_pos, void* out, int n_reqs,
                             int max_q_len, int hidden, int taps, void* stream) {
    if (n_reqs == 0) return 0;
    if (n_reqs < 0 || hidden <= 0 || max_q_len <= 0) RV_FAIL("short_conv: bad sizes");
    if (taps < 1 || taps > RV_CONV_MAX_TAPS)
        RV_FAIL("short_conv: filter length %d is not supported (1 to %d)", taps, RV_CONV_MAX_TAPS);
    if (taps > 1 && !state) RV_FAIL("short_conv: a filter of length %d needs a state", taps);
    const int chunks = (max_q_len + RV_CONV_CHUNK - 1) / RV_CONV_CHUNK;
    if (n_reqs > 65535 || chunks > 65535) RV_FAIL("short_conv: batch too large for one launch");
    const bool aligned = ((uintptr_t)proj % 16 == 0) && ((uintptr_t)out % 16 == 0) &&
                         (!state || (uintptr_t)state % 16 == 0) &&
                         (!in_bias || (uintptr_t)in_bias % 16 == 0) &&
                         (!conv_bias || (uintptr_t)conv_bias % 16 == 0);
    // long portions: the wide kernel (RVLLM_CONV_WIDE_FROM: portions of at least this many tokens)
    static const int wide_from = [] {
        const char* e = getenv("RVLLM_CONV_WIDE_FROM");
        return e && *e ? atoi(e) : 64;
    }();
    if (taps <= RV_CONV_VEC_TAPS && hidden % 8 == 0 && aligned && max_q_len >= wide_from &&
        (uintptr_t)filter % 16 == 0) {
        const int wchunks = (max_q_len + RV_CONV_WIDE_CHUNK - 1) / RV_CONV_WIDE_CHUNK;
        if (wchunks > 65535) RV_FAIL("short_conv: batch too large for one launch");
        dim3 wgrid((hidden / 8 + 127) / 128, n_reqs, wchunks);
        RV_DISPATCH_DTYPE(dtype, "short_conv",
                          (short_conv_wide_launch<T>(wgrid, (cudaStream_t)stream, proj, filter, in_bias,
                                                     conv_bias, state, q_start, state_slot, start_pos,
                                                     out, hidden, taps)));
        RV_CHECK_LAUNCH("short_conv");
        return 0;
    }
    if (taps <= RV_CONV_VEC_TAPS && hidden % 4 == 0 && aligned) {
        dim3 vgrid((hidden / 4 + 127) / 128, n_reqs, chunks);
        RV_DISPATCH_DTYPE(dtype, "short_conv",
                          (rv_launch(short_conv_vec4_kernel<T>, dim3(vgrid), dim3(128), 0,
                                     (cudaStream_t)stream, (const T*)proj, filter, in_bias, conv_bias,
                                     state, q_start, state_slot, start_pos, (T*)out, hidden, taps)));
        RV_CHECK_LAUNCH("short_conv");
        return 0;
    }
    dim3 grid((hidden + 127) / 128, n_reqs, chunks);
    RV_DISPATCH_DTYPE(dtype, "short_conv",
                      (rv_launch(short_conv_kernel<T>, dim3(grid), dim3(128), 0, (cudaStream_t)stream, 
                          (const T*)proj, filter, in_bias, conv_bias, state, q_start, state_slot,
                          start_pos, (T*)out, hidden, taps)));
    RV_CHECK_LAUNCH("short_conv");
    return 0;
}
