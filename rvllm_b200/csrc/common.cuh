// Shared helpers of the sm_100a kernels: storage types, error reporting, reductions.
//
// Every entry point is an `extern "C"` function that takes raw device pointers and a
// stream, validates its sizes, launches, and returns 0 or a non-zero code with a
// message that `rv_last_error()` gives back.  Storage type codes: 0 = float32,
// 1 = bfloat16.  All arithmetic on loaded values is float32.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define RV_DTYPE_F32 0
#define RV_DTYPE_BF16 1

extern "C" const char* rv_last_error();
void rv_set_error(const char* fmt, ...);

#define RV_FAIL(...)                 \
    do {                             \
        rv_set_error(__VA_ARGS__);   \
        return 1;                    \
    } while (0)

#define RV_CHECK_LAUNCH(name)                                                   \
    do {                                                                        \
        cudaError_t e_ = cudaGetLastError();                                    \
        if (e_ != cudaSuccess) RV_FAIL("%s: %s", name, cudaGetErrorString(e_)); \
    } while (0)

// Dispatch a templated launch on the storage type code.
#define RV_DISPATCH_DTYPE(code, name, ...)                       \
    switch (code) {                                              \
        case RV_DTYPE_F32: { using T = float; __VA_ARGS__; break; }          \
        case RV_DTYPE_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
        default: RV_FAIL("%s: unknown dtype code %d", name, (int)(code));    \
    }

__device__ __forceinline__ float rv_load(const float* p) { return *p; }
__device__ __forceinline__ float rv_load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void rv_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void rv_store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float rv_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float rv_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` is shared memory for 33 floats.
__device__ __forceinline__ float rv_block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = rv_warp_sum(v);
    __syncthreads();   // scratch may still be read from a previous call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = rv_warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float rv_block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = rv_warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : -INFINITY;
        t = rv_warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
