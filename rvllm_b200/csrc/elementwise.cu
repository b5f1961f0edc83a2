// Row-wise and element-wise kernels: embedding gather, residual add + RMSNorm,
// SwiGLU activation, bias add.  Plain references: tests/plain_ops.py.
#include <stdarg.h>

#include "common.cuh"

static thread_local char g_error[512] = "";
extern "C" const char* rv_last_error() { return g_error; }
void rv_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

__device__ __forceinline__ float4 rv_load4(const float* p) { return *(const float4*)p; }
__device__ __forceinline__ float4 rv_load4(const __nv_bfloat16* p) {
    const uint2 raw = *(const uint2*)p;
    const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&raw.x);
    const float2 b = __bfloat1622float2(*(const __nv_bfloat162*)&raw.y);
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void rv_store4(float* p, float4 v) { *(float4*)p = v; }
__device__ __forceinline__ void rv_store4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *(const unsigned*)&a;
    raw.y = *(const unsigned*)&b;
    *(uint2*)p = raw;
}

// ---------------------------------------------------------------------------------
// Embedding gather: out[t, :] = table[ids[t], :] (* scale), float32 out.
// Reference counterpart: embed_lookup.cu (one thread per element, float32 table).
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ out, int hidden, int vocab, float scale) {
    rv_pdl_prologue();
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const T* row = table + (size_t)id * hidden;
    float* o = out + (size_t)t * hidden;
    if (hidden % 4 == 0 && ((uintptr_t)table % 16 == 0) && ((uintptr_t)out % 16 == 0)) {
        for (int i = threadIdx.x; i < hidden / 4; i += blockDim.x) {
            const float4 v = rv_load4(row + 4 * i);
            rv_store4(o + 4 * i, make_float4(v.x * scale, v.y * scale, v.z * scale, v.w * scale));
        }
        return;
    }
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = rv_load(row + i) * scale;
}

extern "C" int rv_embed(const void* table, int dtype, const int* ids, float* out, int n_tokens,
                        int hidden, int vocab, float scale, void* stream) {
    if (n_tokens == 0) return 0;
    if (n_tokens < 0 || hidden <= 0 || vocab <= 0) RV_FAIL("embed: bad sizes");
    RV_DISPATCH_DTYPE(dtype, "embed",
                      (rv_launch(embed_kernel<T>, dim3(n_tokens), dim3(hidden >= 2048 ? 512 : 256), 0, (cudaStream_t)stream, 
                          (const T*)table, ids, out, hidden, vocab, scale)));
    RV_CHECK_LAUNCH("embed");
    return 0;
}

// ---------------------------------------------------------------------------------
// Residual add + RMSNorm.  One block per output row; the row is summed into the
// float32 residual stream, kept in shared memory, and normalised:
//   x = resid[r] + delta[r];  out = x / sqrt(mean(x^2) + eps) * w
// With `rows` the block reads row rows[m] and leaves the stream untouched (the final
// norm over the rows whose logits are wanted).
// Without a stream (`resid` null) the rows of `delta` alone are normalised and nothing is
// written back: a norm placed after a sub-layer.
// Reference counterparts: add.cu + rmsnorm.cu + f32_to_f16.cu, three launches.
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                   const float* __restrict__ weight, TO* __restrict__ out,
                                   const int* __restrict__ rows, int hidden, float eps) {
    rv_pdl_prologue();
    extern __shared__ float row[];
    __shared__ float scratch[33];
    const int m = blockIdx.x;
    const size_t in = (size_t)(rows ? rows[m] : m) * hidden;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float x = resid ? resid[in + i] : 0.f;
        if (delta) x += rv_load(delta + in + i);
        if (!rows && delta && resid) resid[in + i] = x;
        row[i] = x;
        ss += x * x;
    }
    const float total = rv_block_sum(ss, scratch);
    const float rms = sqrtf(total / (float)hidden + eps);
    TO* o = out + (size_t)m * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) rv_store(o + i, row[i] / rms * weight[i]);
}

// The same for widths that are a multiple of 4 and at most 16384: every thread keeps up
// to four 4-element chunks of the row in registers, so each global value is loaded once
// with a 16-byte (float32) or 8-byte (bfloat16) access and all loads are in flight together.
template <typename TD, typename TO, int CHUNKS>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                       const float* __restrict__ weight, TO* __restrict__ out,
                                       const int* __restrict__ rows, int hidden, float eps) {
    rv_pdl_prologue();
    __shared__ float scratch[33];
    const int m = blockIdx.x;
    const size_t in = (size_t)(rows ? rows[m] : m) * hidden;
    const int nvec = hidden >> 2;
    float4 x[CHUNKS], w[CHUNKS];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int i = threadIdx.x + c * blockDim.x;
        if (i < nvec) {
            x[c] = resid ? rv_load4(resid + in + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
            w[c] = rv_load4(weight + 4 * i);
            if (delta) {
                const float4 d = rv_load4(delta + in + 4 * i);
                x[c].x += d.x; x[c].y += d.y; x[c].z += d.z; x[c].w += d.w;
                if (!rows && resid) rv_store4(resid + in + 4 * i, x[c]);
            }
            ss += x[c].x * x[c].x + x[c].y * x[c].y + x[c].z * x[c].z + x[c].w * x[c].w;
        }
    }
    const float total = rv_block_sum(ss, scratch);
    const float rms = sqrtf(total / (float)hidden + eps);
    TO* o = out + (size_t)m * hidden;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int i = threadIdx.x + c * blockDim.x;
        if (i < nvec)
            rv_store4(o + 4 * i, make_float4(x[c].x / rms * w[c].x, x[c].y / rms * w[c].y,
                                             x[c].z / rms * w[c].z, x[c].w / rms * w[c].w));
    }
}

template <typename TD, typename TO>
static int add_rmsnorm_launch(float* resid, const void* delta, const float* weight, void* out,
                              const int* rows, int n_rows, int hidden, float eps,
                              cudaStream_t stream) {
    const bool aligned = ((uintptr_t)resid % 16 == 0) && ((uintptr_t)weight % 16 == 0) &&
                         ((uintptr_t)out % 16 == 0) && (!delta || (uintptr_t)delta % 16 == 0);
    if (hidden % 4 == 0 && hidden <= 16384 && aligned) {
        const int nvec = hidden / 4;
        int threads = ((nvec + 31) / 32) * 32;
        int chunks = 1;
        while (threads > 1024 || (chunks < 4 && threads > 512 && nvec > 512)) {
            chunks *= 2;
            threads = (((nvec + chunks - 1) / chunks + 31) / 32) * 32;
        }
        if (chunks == 1)
            rv_launch(add_rmsnorm_vec_kernel<TD, TO, 1>, dim3(n_rows), dim3(threads), 0, stream, 
                resid, (const TD*)delta, weight, (TO*)out, rows, hidden, eps);
        else if (chunks == 2)
            rv_launch(add_rmsnorm_vec_kernel<TD, TO, 2>, dim3(n_rows), dim3(threads), 0, stream, 
                resid, (const TD*)delta, weight, (TO*)out, rows, hidden, eps);
        else
            rv_launch(add_rmsnorm_vec_kernel<TD, TO, 4>, dim3(n_rows), dim3(threads), 0, stream, 
                resid, (const TD*)delta, weight, (TO*)out, rows, hidden, eps);
        RV_CHECK_LAUNCH("add_rmsnorm");
        return 0;
    }
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) RV_FAIL("add_rmsnorm: width %d exceeds the shared-memory row", hidden);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel<TD, TO>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) RV_FAIL("add_rmsnorm: %s", cudaGetErrorString(e));
    }
    const int threads = hidden >= 1024 ? 256 : 128;
    rv_launch(add_rmsnorm_kernel<TD, TO>, dim3(n_rows), dim3(threads), smem, stream, 
        resid, (const TD*)delta, weight, (TO*)out, rows, hidden, eps);
    RV_CHECK_LAUNCH("add_rmsnorm");
    return 0;
}

extern "C" int rv_add_rmsnorm(float* resid, const void* delta, int delta_dtype, const float* weight,
                              void* out, int out_dtype, const int* rows, int n_rows, int hidden,
                              float eps, void* stream) {
    if (n_rows == 0) return 0;
    if (n_rows < 0 || hidden <= 0) RV_FAIL("add_rmsnorm: bad sizes");
    if (!resid && !delta) RV_FAIL("add_rmsnorm: neither a stream nor rows to normalise");
    cudaStream_t s = (cudaStream_t)stream;
    if (delta_dtype == RV_DTYPE_F32 && out_dtype == RV_DTYPE_F32)
        return add_rmsnorm_launch<float, float>(resid, delta, weight, out, rows, n_rows, hidden, eps, s);
    if (delta_dtype == RV_DTYPE_BF16 && out_dtype == RV_DTYPE_BF16)
        return add_rmsnorm_launch<__nv_bfloat16, __nv_bfloat16>(resid, delta, weight, out, rows,
                                                                 n_rows, hidden, eps, s);
    if (delta_dtype == RV_DTYPE_F32 && out_dtype == RV_DTYPE_BF16)
        return add_rmsnorm_launch<float, __nv_bfloat16>(resid, delta, weight, out, rows, n_rows,
                                                        hidden, eps, s);
    if (delta_dtype == RV_DTYPE_BF16 && out_dtype == RV_DTYPE_F32)
        return add_rmsnorm_launch<__nv_bfloat16, float>(resid, delta, weight, out, rows, n_rows,
                                                        hidden, eps, s);
    RV_FAIL("add_rmsnorm: unknown dtype codes %d, %d", delta_dtype, out_dtype);
}

// ---------------------------------------------------------------------------------
// SwiGLU activation: out[n, f] = silu(in[n, f]) * in[n, F + f], silu(z) = z / (1 + e^-z).
// Reference counterpart: silu_gate_multiply.cu (two separate inputs).
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ in, T* __restrict__ out, int ffn, size_t total) {
    rv_pdl_prologue();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / ffn;
        const int f = (int)(i - n * ffn);
        const float g = rv_load(in + n * 2 * ffn + f);
        const float u = rv_load(in + n * 2 * ffn + ffn + f);
        rv_store(out + i, g / (1.f + __expf(-g)) * u);
    }
}

// bfloat16, 8 elements per access (16-byte loads); needs ffn % 8 == 0.  A thread requests the
// gate and up values of two positions before it uses either; index arithmetic is 32-bit when the
// element count allows.
__device__ __forceinline__ uint4 rv_swiglu8(const uint4 g4, const uint4 u4) {
    uint4 o4;
    const __nv_bfloat162* g2 = (const __nv_bfloat162*)&g4;
    const __nv_bfloat162* u2 = (const __nv_bfloat162*)&u4;
    __nv_bfloat162* o2 = (__nv_bfloat162*)&o4;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
        // the quotient is rounded to bfloat16 below: the fast division's last float32 bits do not
        // show (the float32 kernel above divides exactly)
        o2[k] = __floats2bfloat162_rn(__fdividef(g.x, 1.f + __expf(-g.x)) * u.x,
                                      __fdividef(g.y, 1.f + __expf(-g.y)) * u.y);
    }
    return o4;
}

template <typename IDX>
__global__ void swiglu_bf16x8_kernel(const uint4* __restrict__ in, uint4* __restrict__ out,
                                     int ffn8, size_t total8) {
    rv_pdl_prologue();
    const IDX step = (IDX)gridDim.x * blockDim.x, n8 = (IDX)total8, f8 = (IDX)ffn8;
    for (IDX i = (IDX)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += 2 * step) {
        const IDX j = i + step;
        const bool two = j < n8;
        const IDX ni = i / f8, nj = two ? j / f8 : ni;
        const IDX pi = ni * f8 + i, pj = two ? nj * f8 + j : pi;      // = n * 2 * ffn8 + f
        const uint4 gi = in[pi], ui = in[pi + f8], gj = in[pj], uj = in[pj + f8];
        out[i] = rv_swiglu8(gi, ui);
        if (two) out[j] = rv_swiglu8(gj, uj);
    }
}

extern "C" int rv_swiglu(const void* in, void* out, int dtype, int n_rows, int ffn, void* stream) {
    if (n_rows == 0) return 0;
    if (n_rows < 0 || ffn <= 0) RV_FAIL("swiglu: bad sizes");
    const size_t total = (size_t)n_rows * ffn;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RV_DTYPE_BF16 && ffn % 8 == 0 && ((uintptr_t)in % 16 == 0) &&
        ((uintptr_t)out % 16 == 0)) {
        const size_t total8 = total / 8;
        const int blocks = (int)((total8 + 255) / 256 < 148 * 16 ? (total8 + 255) / 256 : 148 * 16);
        if (total8 * 2 < 0x7fffffffull)
            rv_launch(swiglu_bf16x8_kernel<unsigned>, dim3(blocks), dim3(256), 0, s, (const uint4*)in,
                      (uint4*)out, ffn / 8, total8);
        else
            rv_launch(swiglu_bf16x8_kernel<size_t>, dim3(blocks), dim3(256), 0, s, (const uint4*)in,
                      (uint4*)out, ffn / 8, total8);
    } else {
        const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
        RV_DISPATCH_DTYPE(dtype, "swiglu",
                          (rv_launch(swiglu_kernel<T>, dim3(blocks), dim3(256), 0, s, (const T*)in, (T*)out, ffn, total)));
    }
    RV_CHECK_LAUNCH("swiglu");
    return 0;
}

// ---------------------------------------------------------------------------------
// x[n, :] += bias (float32 bias).  Reference counterpart: add_bias.cu.
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, const float* __restrict__ bias, int width,
                                size_t total) {
    rv_pdl_prologue();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x)
        rv_store(x + i, rv_load(x + i) + bias[i % width]);
}

extern "C" int rv_add_bias(void* x, int dtype, const float* bias, int n_rows, int width,
                           void* stream) {
    if (n_rows == 0) return 0;
    if (n_rows < 0 || width <= 0) RV_FAIL("add_bias: bad sizes");
    const size_t total = (size_t)n_rows * width;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    RV_DISPATCH_DTYPE(dtype, "add_bias",
                      (rv_launch(add_bias_kernel<T>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, 
                          (T*)x, bias, width, total)));
    RV_CHECK_LAUNCH("add_bias");
    return 0;
}
