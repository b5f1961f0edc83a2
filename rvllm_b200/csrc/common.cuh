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
#include <stdlib.h>

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

// ---- programmatic dependent launch -------------------------------------------------------
// Every kernel of this library is launched with the programmatic-stream-serialization
// attribute and begins with `rv_pdl_prologue()`: it lets the next kernel of the stream
// start (and run whatever it does before its own wait, e.g. the matrix product's copies
// of weight tiles), then waits until the previous kernel has completed and its writes
// are visible.  Before the wait a kernel reads only what no kernel of the same step writes:
// constant weights and tables and the step's index arrays (positions, slots, block tables,
// context lengths: copied from the host before the step's first kernel); it writes nothing.
// (Not even state that "only this layer" writes: a run order may name a layer twice, and
// several short kernels can be resident and waiting at once.)  A few
// kernels therefore split the prologue into `rv_pdl_launch_dependents()`, those loads, and
// `rv_pdl_wait()`.  RVLLM_PDL=0 turns the attribute off (the two instructions are then
// no-ops).
__device__ __forceinline__ void rv_pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::);
}
__device__ __forceinline__ void rv_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void rv_pdl_prologue() {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
}
// Streaming multiprocessors of the current device (asked once per device).
static inline int rv_sm_count() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (cached[dev] <= 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}
static inline int rv_pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("RVLLM_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v;
}
template <typename... KArgs, typename... Args>
static inline void rv_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = rv_pdl_enabled();
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
