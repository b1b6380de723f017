// Tensor-pipe rate probe: how fast does this GPU retire tcgen05.mma instructions when nothing
// else is in the way? Every SM runs one CTA whose single issuing thread streams MMAs of the
// largest shape (M 128, N 256) on operands that already sit in shared / tensor memory; no data
// moves. The result is the denominator for "fraction of the tensor pipe" figures where no
// library GEMM exists to measure against (block-scaled NVFP4), and a cross-check of the bf16
// figure. Operands are a constant fill: only the timing is used.
// No reference counterpart.
#include <cuda_runtime.h>

#include <cstdint>

#include "common.cuh"
#include "kernels.h"

namespace xmoe {

namespace {

constexpr int kProbeThreads = 64;
constexpr int kProbeSmem = 1024 + 16384 + 32768;  // A tile (128 x 128 B) + B tile (256 x 128 B), 128-byte swizzle
constexpr int kPerCommit = 64;

// KIND 0: NVFP4 block-scaled (K 64 per MMA), 1: bf16 (K 16 per MMA)
template <int KIND>
__global__ __launch_bounds__(kProbeThreads, 1) void mma_rate_kernel(int n_mma, uint32_t* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    __shared__ uint32_t abort_word;
    volatile uint32_t* abort_flag = &abort_word;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // finite operands (every byte 0x22) rather than whatever shared memory held
    for (int i = threadIdx.x; i < (16384 + 32768) / 16; i += blockDim.x)
        reinterpret_cast<uint4*>(smem)[i] = make_uint4(0x22222222u, 0x22222222u, 0x22222222u, 0x22222222u);
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_word = 0u;
        mbar_fence_init();
    }
    fence_proxy_async_smem();
    if (warp == 0) {
        tmem_alloc(&tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    if (warp == 1 && lane == 0) {
        const uint32_t a_lo = umma_desc_lo_sw128(smem_u32(smem));
        const uint32_t b_lo = umma_desc_lo_sw128(smem_u32(smem + 16384));
        uint32_t parity = 0;
        if (KIND == 0) {  // finite scale factors (UE4M3 0x22) for A (4 columns) and B (8 columns)
            const uint32_t sf_lo = umma_desc_lo_sf(smem_u32(smem));
            tmem_cp_sf_lo(tmem_base + 256, sf_lo);
            tmem_cp_sf_lo(tmem_base + 272, sf_lo + 32);
            tmem_cp_sf_lo(tmem_base + 276, sf_lo + 64);
        }
        for (int i = 0; i < n_mma; i += kPerCommit) {
#pragma unroll 4
            for (int k = 0; k < kPerCommit; ++k) {
                if (KIND == 0) {
                    constexpr uint32_t idesc = umma_idesc_nvfp4(128, 256);
                    mma_nvfp4_lo(tmem_base, a_lo + (k & 3) * 2, b_lo + (k & 3) * 2, idesc, tmem_base + 256,
                                 tmem_base + 272, 1u);
                } else {
                    constexpr uint32_t idesc = umma_idesc_bf16(128, 256);
                    mma_bf16(tmem_base, ((uint64_t)kDescHiSw128 << 32) | (a_lo + (k & 3) * 2),
                             ((uint64_t)kDescHiSw128 << 32) | (b_lo + (k & 3) * 2), idesc, 1u);
                }
            }
            tc_commit(&bar);
            if (!mbar_wait(&bar, parity, abort_flag, status, XMOE_DEV_TIMEOUT_MMA)) break;
            parity ^= 1u;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, 512);
}

template <int KIND>
int run_probe(int n_mma, int grid, uint32_t* status, float* ms_out, cudaStream_t stream) {
    if (cudaFuncSetAttribute(mma_rate_kernel<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, kProbeSmem) !=
        cudaSuccess)
        return XMOE_ERR_CUDA;
    cudaEvent_t e0, e1;
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return XMOE_ERR_CUDA;
    int rc = XMOE_OK;
    for (int rep = 0; rep < 3 && rc == XMOE_OK; ++rep) {  // the last repetition is the one reported
        cudaEventRecord(e0, stream);
        mma_rate_kernel<KIND><<<grid, kProbeThreads, kProbeSmem, stream>>>(n_mma, status);
        cudaEventRecord(e1, stream);
        if (cudaGetLastError() != cudaSuccess || cudaEventSynchronize(e1) != cudaSuccess) rc = XMOE_ERR_CUDA;
    }
    if (rc == XMOE_OK && cudaEventElapsedTime(ms_out, e0, e1) != cudaSuccess) rc = XMOE_ERR_CUDA;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return rc;
}

}  // namespace

int probe_mma_rate(int kind, int n_mma, double* tflops_out, cudaStream_t stream) {
    if (!tflops_out || n_mma < kPerCommit || (kind != 0 && kind != 1)) return XMOE_ERR_ARG;
    n_mma = n_mma / kPerCommit * kPerCommit;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
        return XMOE_ERR_CUDA;
    uint32_t* status = nullptr;
    if (cudaMalloc(&status, 4) != cudaSuccess) return XMOE_ERR_CUDA;
    cudaMemsetAsync(status, 0, 4, stream);
    float ms = 0.f;
    int rc = kind == 0 ? run_probe<0>(n_mma, sms, status, &ms, stream) : run_probe<1>(n_mma, sms, status, &ms, stream);
    uint32_t st = 0;
    if (rc == XMOE_OK && cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost) != cudaSuccess) rc = XMOE_ERR_CUDA;
    cudaFree(status);
    if (rc != XMOE_OK) return rc;
    if (st != XMOE_DEV_OK) return XMOE_ERR_TIMEOUT;
    const double flop_per_mma = 2.0 * 128.0 * 256.0 * (kind == 0 ? 64.0 : 16.0);
    *tflops_out = flop_per_mma * (double)n_mma * (double)sms / ((double)ms * 1e-3) * 1e-12;
    return XMOE_OK;
}

}  // namespace xmoe
