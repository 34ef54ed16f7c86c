// Ceiling of the integer tensor pipe as this library drives it: tcgen05.mma kind::i8 issued back to back on
// operands that already sit in shared memory (no TMA, no epilogue), one CTA -- or CTA pair -- per SM.  The
// distance kernels are compared with this figure beside the nominal one.
#include "../../include/pink_b200.h"
#include "kernels.cuh"
#include "ptx.cuh"

namespace pinkb {

template <bool PAIR>
__global__ void __launch_bounds__(128, 1) mma_peak_kernel(uint32_t iters, uint32_t n, int* status)
{
    extern __shared__ uint8_t raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t done_bar;
    __shared__ uint32_t tmem_ptr;
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0;
    // one 128-row A slice (16 KB) and one 256-row B slice (32 KB) of 128 bytes of K; the values do not matter
    for (uint32_t i = threadIdx.x; i < (16384 + 32768) / 4; i += 128) reinterpret_cast<uint32_t*>(smem)[i] = i * 2654435761u;
    if (threadIdx.x == 0) { mbar_init(&done_bar, 1); mbar_fence_init(); }
    if (warp == 1) {
        if (PAIR) { tmem_alloc_pair(&tmem_ptr, 256); tmem_relinquish_pair(); }
        else { tmem_alloc(&tmem_ptr, 256); tmem_relinquish(); }
    }
    fence_async_smem();
    tc_fence_before();
    if (PAIR) cluster_sync(); else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_ptr;
    if (warp == 0 && rank == 0 && elect_one()) {
        const uint32_t idesc = make_idesc_u8(PAIR ? 256 : 128, n);
        const uint64_t a = make_sw128_kmajor_desc(smem_u32(smem)), b = make_sw128_kmajor_desc(smem_u32(smem + 16384));
        for (uint32_t i = 0; i < iters; ++i) {
#pragma unroll
            for (uint32_t k = 0; k < 4; ++k) {
                if (PAIR) umma_i8_pair(tmem_base, a + 2 * k, b + 2 * k, idesc, 1u);
                else umma_i8(tmem_base, a + 2 * k, b + 2 * k, idesc, 1u);
            }
        }
        if (PAIR) { umma_commit_pair(smem_u32(&done_bar)); umma_commit_pair(map_to_cta(smem_u32(&done_bar), 1)); }
        else umma_commit(&done_bar);
    }
    if (!mbar_wait(&done_bar, 0)) atomicExch(status, kDevTimeoutMma);      // bounded wait: reports instead of hanging
    tc_fence_before();
    if (PAIR) cluster_sync(); else __syncthreads();
    if (warp == 1) { if (PAIR) tmem_dealloc_pair(tmem_base, 256); else tmem_dealloc(tmem_base, 256); }
}

template <bool PAIR> static int run_peak(uint32_t n, double* tops)
{
    int sms = 0, dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return PINK_B200_ECUDA;
    const int ctas = PAIR ? (sms & ~1) : sms;
    const uint32_t iters = 4096;
    const int smem = 64 * 1024;
    int* status = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    int rc = PINK_B200_OK;
    double best = 0.0;
    if (cudaMalloc(&status, sizeof(int)) != cudaSuccess) return PINK_B200_ECUDA;
    if (cudaMemset(status, 0, sizeof(int)) != cudaSuccess || cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess ||
        cudaFuncSetAttribute(mma_peak_kernel<PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) rc = PINK_B200_ECUDA;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas); cfg.blockDim = dim3(128); cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = PAIR ? 2 : 1; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    for (int rep = 0; rep < 4 && rc == PINK_B200_OK; ++rep) {            // the first launch warms up
        float ms = 0.f;
        int st = 0;
        if (cudaEventRecord(e0) != cudaSuccess || cudaLaunchKernelEx(&cfg, mma_peak_kernel<PAIR>, iters, n, status) != cudaSuccess ||
            cudaEventRecord(e1) != cudaSuccess || cudaEventSynchronize(e1) != cudaSuccess || cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess ||
            cudaMemcpy(&st, status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) { rc = PINK_B200_ECUDA; break; }
        if (st != 0) { rc = PINK_B200_ETIMEOUT; break; }
        const double ops = 2.0 * 128.0 * n * 32.0 * 4.0 * iters * ctas;     // each CTA's share: 128 rows x n columns x 32 of K per instruction
        if (rep > 0 && ms > 0.f) best = ops / (ms * 1e-3) / 1e12 > best ? ops / (ms * 1e-3) / 1e12 : best;
    }
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(status);
    if (rc == PINK_B200_OK) *tops = best;
    return rc;
}

}  // namespace pinkb

extern "C" int pink_b200_mma_i8_peak(int device, uint32_t n, int pair, double* tops)
{
    if (!tops || n < 16 || n > 256 || (n % 16) != 0) return PINK_B200_EINVAL;
    if (cudaSetDevice(device) != cudaSuccess) return PINK_B200_ECUDA;
    return pair ? pinkb::run_peak<true>(n, tops) : pinkb::run_peak<false>(n, tops);
}
