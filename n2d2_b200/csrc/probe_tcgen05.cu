// Issue-rate probe of the int8 tensor pipe: every SM runs one CTA whose single issuing thread sends
// tcgen05.mma kind::i8 instructions (M = 128, K = 32, N as given) back to back from operands that sit
// in shared memory, alternating between two TMEM accumulators.  No memory traffic, no epilogue: the
// time of the launch is what the tensor pipe itself needs, i.e. the denominator a convolution kernel's
// achieved TOP/s is to be compared with on this very GPU at the clocks it holds under this load.
#include <cstdio>
#include <cstring>
#include "../../include/n2d2b.h"
#include "host_internal.h"
#include "tc_common.cuh"

namespace n2d2b {

__global__ void __launch_bounds__(128, 1) mma_rate_probe_kernel(int N, int reps, long long* cycles, int* status)
{
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* smA = smem;              // 128 rows x 128 bytes, 128-byte swizzle
    unsigned char* smB = smem + 16384;      // 256 rows x 128 bytes
    __shared__ unsigned long long bar;
    __shared__ unsigned tmem_slot;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < 16384 + 32768; i += 128) smem[i] = (unsigned char)(i * 7 + 3);
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fence_async_smem();
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = tmem_slot;
    if (threadIdx.x == 0) {
        const unsigned idesc = (2u << 4) | (0u << 7) | (1u << 10) | (((unsigned)N >> 3) << 17) | ((128u >> 4) << 24);
        const unsigned desc_hi = (unsigned)(make_smem_desc(0u, 128) >> 32);
        const unsigned a_lo = (smem_u32(smA) & 0x3ffffu) >> 4, b_lo = (smem_u32(smB) & 0x3ffffu) >> 4;
        const long long t0 = clock64();
#pragma unroll 4
        for (int r = 0; r < reps; ++r) {
            const unsigned d = tmem + (unsigned)((r & 1) * N);
            const unsigned k = 2u * (unsigned)(r & 3);
            tc_mma_i8_lohi(d, a_lo + k, b_lo + k, desc_hi, idesc, 1u);
        }
        tc_commit(smem_u32(&bar));
        mbar_wait(smem_u32(&bar), 0, &abort_flag, status, 10);
        if (blockIdx.x == 0) cycles[0] = clock64() - t0;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

}  // namespace n2d2b

extern "C" int n2d2b_probe_i8_mma_rate(int device, int n, int reps, double* tops, double* cycles_per_mma)
{
    using namespace n2d2b;
    if (!tops || !cycles_per_mma) return set_error(N2D2B_ERR_INVALID, "result pointers must not be NULL");
    if (n < 16 || n > 256 || n % 16) return set_error(N2D2B_ERR_INVALID, "n must be a multiple of 16 in 16..256");
    if (reps < 64 || reps > 1000000) return set_error(N2D2B_ERR_INVALID, "reps must be in 64..1000000");
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return set_error(N2D2B_ERR_CUDA, "cudaSetDevice(%d) failed: %s", device, cudaGetErrorString(e));
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (sms < 1) return set_error(N2D2B_ERR_CUDA, "no multiprocessors reported for device %d", device);
    long long* d_cycles = nullptr;
    int* d_status = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    int rc = 0;
    float ms = 0.0f;
    long long cyc = 0;
    int st = 0;
#define PROBE_TRY(expr)                                                                               \
    if (rc == 0 && (e = (expr)) != cudaSuccess)                                                       \
        rc = set_error(N2D2B_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e))
    PROBE_TRY(cudaMalloc(&d_cycles, 64));
    PROBE_TRY(cudaMalloc(&d_status, 64));
    PROBE_TRY(cudaMemset(d_status, 0, 64));
    PROBE_TRY(cudaMemset(d_cycles, 0, 64));
    PROBE_TRY(cudaFuncSetAttribute(mma_rate_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
    PROBE_TRY(cudaEventCreate(&e0));
    PROBE_TRY(cudaEventCreate(&e1));
    if (rc == 0) {
        // one short untimed launch (module load, clocks), then the timed one
        mma_rate_probe_kernel<<<sms, 128, 60 * 1024>>>(n, 256, d_cycles, d_status);
        PROBE_TRY(cudaEventRecord(e0, 0));
        mma_rate_probe_kernel<<<sms, 128, 60 * 1024>>>(n, reps, d_cycles, d_status);
        PROBE_TRY(cudaEventRecord(e1, 0));
        PROBE_TRY(cudaEventSynchronize(e1));
        PROBE_TRY(cudaEventElapsedTime(&ms, e0, e1));
        PROBE_TRY(cudaMemcpy(&cyc, d_cycles, sizeof(cyc), cudaMemcpyDeviceToHost));
        PROBE_TRY(cudaMemcpy(&st, d_status, sizeof(st), cudaMemcpyDeviceToHost));
    }
#undef PROBE_TRY
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(d_cycles);
    cudaFree(d_status);
    if (rc) return rc;
    if (st != 0) return set_error(N2D2B_ERR_TIMEOUT, "the probe's completion wait gave up");
    if (ms <= 0.0f) return set_error(N2D2B_ERR_CUDA, "the probe measured no time");
    *tops = 2.0 * 128.0 * n * 32.0 * (double)reps * sms / (ms * 1e-3) / 1e12;
    *cycles_per_mma = (double)cyc / reps;
    return 0;
}
