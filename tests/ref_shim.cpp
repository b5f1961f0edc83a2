// Runs the reference project's CUDA kernel sources on the CPU, unchanged.
//
// The reference (ermolushka/rvllm) keeps its device code as small `.cu` files under
// src/cuda/kernels/.  They use nothing of CUDA but the thread indices, `__syncthreads`,
// shared memory and a few math functions, so they compile as plain C++ once those names
// exist.  This file defines the names, `#include`s the sources from the reference checkout
// (its kernels folder is given to the compiler with -I; nothing is copied into this
// repository) and exports one `run_<kernel>` function per kernel that walks the launch grid
// with ordinary loops.
//
// Kernels that reduce over a block (rmsnorm, softmax, argmax) are launched with one thread
// per block: their strided loops then cover the whole row, their tree reductions have no
// step to take, and `__syncthreads` has nobody to wait for.  That exercises each kernel's
// formula, which is what the tests compare with; the parallel reduction itself is not
// under test.
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>

struct Dim3 { unsigned int x = 1, y = 1, z = 1; };
static thread_local Dim3 blockIdx, blockDim, threadIdx, gridDim;

#define __global__
#define __device__ static inline
// Static shared variables (`__shared__ float rms;`) become locals of the one thread that
// runs the block.  The dynamic shared memory of a launch (`extern __shared__ float
// sdata[];`, `extern __shared__ unsigned char smem[];`) becomes a declaration of the two
// arrays defined below.
#define __shared__
static inline void __syncthreads() {}
static inline float __int_as_float(int bits) {
    float f;
    std::memcpy(&f, &bits, sizeof f);
    return f;
}
extern "C" {
float sdata[1 << 16];
unsigned char smem[1 << 18];
}

// ---- the reference's sources, compiled as they are (found through -I) ----------------------
#include "short_conv.cu"
#include "rope.cu"
#include "silu_gate_multiply.cu"
#include "rmsnorm.cu"
#include "softmax.cu"
#include "argmax.cu"
#include "kv_write.cu"
#include "kv_gather.cu"
#include "embed_lookup.cu"

namespace ref {
using ::short_conv_bx; using ::short_conv_filter_gate; using ::rope; using ::silu_gate_multiply;
using ::rmsnorm; using ::softmax; using ::argmax; using ::kv_write; using ::kv_gather;
using ::embed_lookup;
}   // namespace ref

template <typename F>
static void launch(unsigned int blocks, unsigned int threads, F body) {
    gridDim.x = blocks;
    blockDim.x = threads;
    for (unsigned int b = 0; b < blocks; ++b) {
        blockIdx.x = b;
        for (unsigned int t = 0; t < threads; ++t) {
            threadIdx.x = t;
            body();
        }
    }
}

static unsigned int blocks_for(unsigned int n, unsigned int threads) { return (n + threads - 1) / threads; }

extern "C" {

void run_short_conv_bx(const float* proj, float* bx, unsigned int hidden, unsigned int n) {
    launch(blocks_for(n, 256), 256, [&] { ref::short_conv_bx(proj, bx, hidden, n); });
}

void run_short_conv_filter_gate(const float* window, const float* filter, const float* proj,
                                float* out, unsigned int batch, unsigned int q_len,
                                unsigned int hidden, unsigned int kernel) {
    const unsigned int n = batch * q_len * hidden;
    launch(blocks_for(n, 256), 256, [&] {
        ref::short_conv_filter_gate(window, filter, proj, out, batch, q_len, hidden, kernel, n);
    });
}

void run_rope(const float* x, const float* cos_t, const float* sin_t, float* out,
              unsigned int head_dim, unsigned int rows) {
    const unsigned int half = head_dim / 2, n = rows * half;
    launch(blocks_for(n, 128), 128, [&] { ref::rope(x, cos_t, sin_t, out, head_dim, half, n); });
}

void run_silu_gate_multiply(const float* gate, const float* up, float* out, unsigned int n) {
    launch(blocks_for(n, 256), 256, [&] { ref::silu_gate_multiply(gate, up, out, n); });
}

void run_rmsnorm(const float* x, const float* weight, float* out, unsigned int rows,
                 unsigned int hidden, float eps) {
    launch(rows, 1, [&] { ref::rmsnorm(x, weight, out, hidden, eps); });
}

void run_softmax(const float* x, float* out, unsigned int rows, unsigned int row_len) {
    launch(rows, 1, [&] { ref::softmax(x, out, row_len); });
}

void run_argmax(const float* x, unsigned int* out, unsigned int rows, unsigned int row_len) {
    launch(rows, 1, [&] { ref::argmax(x, out, row_len); });
}

void run_kv_write(const float* k, const float* v, const unsigned int* block_ids,
                  const unsigned int* offsets, float* out_k, float* out_v,
                  unsigned int n_tokens, unsigned int n_kv_heads, unsigned int head_dim,
                  unsigned int block_size) {
    const unsigned int n = n_tokens * n_kv_heads * head_dim;
    launch(blocks_for(n, 256), 256, [&] {
        ref::kv_write(k, v, block_ids, offsets, out_k, out_v, n_kv_heads, head_dim, block_size, n);
    });
}

void run_kv_gather(const float* cache, const unsigned int* block_idx, float* out,
                   unsigned int batch, unsigned int max_blocks, unsigned int ctx_len,
                   unsigned int block_size, unsigned int n_kv_heads, unsigned int head_dim) {
    const unsigned int n = batch * n_kv_heads * ctx_len * head_dim;
    launch(blocks_for(n, 256), 256, [&] {
        ref::kv_gather(cache, block_idx, out, batch, max_blocks, ctx_len, block_size, n_kv_heads,
                       head_dim, n);
    });
}

void run_embed_lookup(const unsigned int* ids, const float* table, float* out,
                      unsigned int n_tokens, unsigned int hidden) {
    const unsigned int n = n_tokens * hidden;
    launch(blocks_for(n, 256), 256, [&] { ref::embed_lookup(ids, table, out, hidden, n); });
}

}   // extern "C"
