// A measuring probe, not part of any step: how fast blocks can copy 16 KB tiles from device
// memory into a ring in shared memory, (0) as 2-D tensor-map boxes [128 rows x 64 bfloat16] of
// a row-major [rows, K] matrix, the way the weight-streaming product copies its tiles, or (1) as
// 1-D bulk copies of 16 KB contiguous.  Nothing consumes the tiles: a stage is reused as soon as
// its copy has arrived, so the time is that of the copies alone.  With one block per SM and
// fewer blocks than SMs it gives the copy rate a single SM can sustain, which bounds every
// kernel of this library that streams weights through TMA (measured on a B200: about 52 GB/s per
// SM for boxes and 70 GB/s for bulk copies, whatever the ring's depth; 6.3 to 6.9 TB/s with all
// 148 SMs, where HBM is the limit).  `bench.py --only kernels --kernel copy_rate` runs it.
#include "tcgen05_common.cuh"

__global__ void __launch_bounds__(64, 1)
copy_probe_kernel(const __grid_constant__ CUtensorMap map, const char* flat, int mode, int iters,
                  int stages, int kblocks, int chunk, int* status) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* ring = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ unsigned long long full[16];
    __shared__ volatile int failed;
    if (threadIdx.x == 0) {
        failed = 0;
        for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    for (int i = 0; i < iters + stages; ++i) {
        const int s = i % stages;
        if (i >= stages && !mbar_wait(&full[s], (unsigned)((i / stages) - 1) & 1u, &failed)) {
            atomicCAS(status, 0, 41);        // the copy issued `stages` iterations ago never arrived
            return;
        }
        if (i < iters) {
            mbar_expect_tx(&full[s], (unsigned)chunk);
            const long long item = (long long)blockIdx.x * iters + i;
            if (mode == 0)
                tma_load_2d(ring + (size_t)s * chunk, &map, &full[s], (int)(item % kblocks) * 64,
                            (int)(item / kblocks) * 128);
            else
                bulk_load_1d(ring + (size_t)s * chunk, flat + item * chunk, (unsigned)chunk, &full[s]);
        }
    }
}

// `w`: [rows, K] bfloat16 with rows * K * 2 >= grid * iters * 16384 bytes.
// `chunk`: bytes per copy (16384 for boxes; for bulk copies any multiple of 16 up to 65536).
extern "C" int rv_copy_probe(const void* w, long long rows, int K, int mode, int grid, int iters,
                             int stages, int chunk, int* status, void* stream) {
    if (K % 64 || stages < 1 || stages > 12 || grid < 1 || iters < 1 || (mode != 0 && mode != 1))
        RV_FAIL("copy_probe: bad arguments");
    if (chunk % 16 || chunk < 16 || chunk > 65536 || (mode == 0 && chunk != 16384) ||
        (size_t)stages * chunk > 200 * 1024)
        RV_FAIL("copy_probe: bad chunk size %d", chunk);
    if ((long long)grid * iters * chunk > rows * K * 2) RV_FAIL("copy_probe: the matrix is too small");
    CUtensorMap map;
    if (make_map(&map, w, rows, K, 128)) return 1;
    const size_t smem = (size_t)stages * chunk + 1024;
    cudaError_t e = cudaFuncSetAttribute(copy_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) RV_FAIL("copy_probe: %s", cudaGetErrorString(e));
    copy_probe_kernel<<<grid, 64, smem, (cudaStream_t)stream>>>(map, (const char*)w, mode, iters, stages,
                                                                K / 64, chunk, status);
    RV_CHECK_LAUNCH("copy_probe");
    return 0;
}
