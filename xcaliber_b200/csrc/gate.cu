// Router gate GEMM: logits[N, E] = x[N, H] @ Wr[E, H]^T, bf16 inputs, fp32 accumulation, bf16 output.
//
// The step immediately before the layer. In the reference (and in vLLM) it runs outside the
// operator (vllm/xcaliber_int4_vllm/method.py:255-257 receives router_logits ready-made);
// xmoe_forward_gated runs it here so that a caller hands over x and the gate weight only.
//
// One CTA per 128 tokens: tcgen05.mma kind::f16 with the token tile as the M operand and the
// gate rows as N (E rounded up to 16, at most 256), both staged by TMA with the 128-byte swizzle,
// K 64 per stage. The accumulator (128 lanes x N columns of tensor memory) is read back by four
// warps, lane = token, and stored as bf16 rows. Every wait is bounded.
//
// ROUTE != 0 (xmoe_forward_gated): the same kernel also routes. Each epilogue warp rounds the logits of its
// 32 tokens to bf16 into a shared-memory tile (the pipeline stages are free by then) and then runs the
// router's own per-token routine (router_core.cuh, one warp per token) on those rows: top-k indices and gate
// weights go straight to the layer's workspace, the same bits as the gate GEMM followed by the router kernel,
// and the logits need not touch HBM at all (they are stored only when the caller passes a buffer).
#include <cuda_bf16.h>

#include "common.cuh"
#include "kernels.h"
#include "router_core.cuh"

namespace xmoe {

namespace {

constexpr int kGateM = 128;
constexpr int kGateStages = 4;
constexpr int kGateThreads = 192;  // producer warp, MMA warp, 4 epilogue warps
constexpr int kGateABytes = kGateM * 128;

// ROUTE: 0 logits only, 1 flat softmax top-k, 2 flat sigmoid top-k, 3 group-limited sigmoid top-k
template <int ROUTE>
__global__ __launch_bounds__(kGateThreads, 1) void gate_logits_kernel(const __grid_constant__ CUtensorMap tm_x,
                                                                     const __grid_constant__ CUtensorMap tm_w,
                                                                     uint16_t* __restrict__ logits, int n, int E, int H,
                                                                     int n_pad, int x_box_rows, int w_box_rows,
                                                                     uint32_t* status, const RouterArgs r) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int b_bytes = n_pad * 128;
    const int stage_bytes = kGateABytes + b_bytes;
    uint8_t* tail = smem + (size_t)kGateStages * stage_bytes;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);
    uint64_t* empty_bar = full_bar + 8;
    uint64_t* acc_full = empty_bar + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_stages = H / 64;
    const int row0 = blockIdx.x * kGateM;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kGateStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0u;
        mbar_fence_init();
        prefetch_tmap(&tm_x);
        prefetch_tmap(&tm_w);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int ks = 0; ks < k_stages; ++ks) {
                const int s = ks % kGateStages;
                const uint32_t ph = (ks / kGateStages) & 1u;
                if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, status, XMOE_DEV_TIMEOUT_MMA)) break;
                uint8_t* st = smem + (size_t)s * stage_bytes;
                mbar_expect_tx(&full_bar[s], (uint32_t)(x_box_rows + w_box_rows) * 128u);
                tma_load_2d(st, &tm_x, ks * 64, row0, &full_bar[s]);
                tma_load_2d(st + kGateABytes, &tm_w, ks * 64, 0, &full_bar[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(kGateM, (uint32_t)n_pad);
            bool ok = true;
            for (int ks = 0; ks < k_stages && ok; ++ks) {
                const int s = ks % kGateStages;
                const uint32_t ph = (ks / kGateStages) & 1u;
                if (!mbar_wait(&full_bar[s], ph, abort_flag, status, XMOE_DEV_TIMEOUT_TMA)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + (size_t)s * stage_bytes);
                const uint64_t a_desc = umma_desc_sw128(a_addr);
                const uint64_t b_desc = umma_desc_sw128(a_addr + kGateABytes);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)  // 32 bytes of K per MMA inside the 128-byte swizzle row
                    mma_bf16(tmem_base, a_desc + kk * 2, b_desc + kk * 2, idesc, (ks | kk) ? 1u : 0u);
                tc_commit(&empty_bar[s]);
            }
            if (ok) tc_commit(acc_full);
        }
    } else {
        const int q = warp & 3;  // tensor-memory lane quadrant of this warp
        if (mbar_wait(acc_full, 0u, abort_flag, status, XMOE_DEV_TIMEOUT_ACC)) {
            tc_fence_after();
            const int t = row0 + q * 32 + lane;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
            // ROUTE: this warp's 32 x E bf16 logits, row pitch n_pad + 2 (odd in 32-bit words: the lanes' 2-byte
            // stores of one column fall into 32 different banks). All MMAs have retired: the stages are free.
            const int pitch = n_pad + 2;
            uint16_t* tile = reinterpret_cast<uint16_t*>(smem) + (size_t)q * 32 * pitch;
            for (int c0 = 0; c0 < n_pad; c0 += 16) {
                uint32_t v[16];
                tmem_ld16(lane_addr + c0, v);
                tmem_ld_wait();
                if (ROUTE) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) tile[lane * pitch + c0 + j] = (uint16_t)f32_to_bf16_bits(__uint_as_float(v[j]));
                }
                if (logits && t < n) {
                    uint16_t* dst = logits + (size_t)t * E + c0;
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (c0 + j < E) dst[j] = (uint16_t)f32_to_bf16_bits(__uint_as_float(v[j]));
                }
            }
            if (ROUTE) {
                __syncwarp();
                const uint16_t* es = reinterpret_cast<const uint16_t*>(r.expert_scale);
                uint16_t* tw = reinterpret_cast<uint16_t*>(r.topk_w);
                for (int i = 0; i < 32; ++i) {
                    const int token = row0 + q * 32 + i;
                    if (token >= n) break;  // uniform across the warp
                    const uint16_t* row = tile + i * pitch;
                    if (ROUTE == 1)
                        route_token_flat<false, 8>(row, (uint32_t)lane, (uint32_t)token, es, r.topk_idx, tw, E, r.topk,
                                                r.idx_stride, r.routed_scale, r.renorm);
                    else if (ROUTE == 2)
                        route_token_flat<true, 8>(row, (uint32_t)lane, (uint32_t)token, es, r.topk_idx, tw, E, r.topk,
                                               r.idx_stride, r.routed_scale, r.renorm);
                    else
                        route_token_grouped<8>(row, (uint32_t)lane, (uint32_t)token, r.lut, r.bias, es, r.topk_idx, tw, E,
                                               r.topk, r.idx_stride, r.n_group, r.topk_group, r.routed_scale, r.renorm);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 256);
}

}  // namespace

namespace {
template <int ROUTE>
int launch_gate_t(const CUtensorMap& tm_x, const CUtensorMap& tm_w, void* logits, int n, int E, int H, int n_pad,
                  int x_box_rows, int w_box_rows, uint32_t* status, const RouterArgs& r, cudaStream_t stream) {
    const size_t smem = 1024 + (size_t)kGateStages * (kGateABytes + (size_t)n_pad * 128) + 256;
    static size_t configured_dev[kMaxDevices] = {};
    const int dev = device_slot();
    if (dev < 0) return XMOE_ERR_CUDA;
    size_t& configured = configured_dev[dev];
    if (smem > configured) {
        if (cudaFuncSetAttribute(gate_logits_kernel<ROUTE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return XMOE_ERR_CUDA;
        configured = smem;
    }
    gate_logits_kernel<ROUTE><<<(n + kGateM - 1) / kGateM, kGateThreads, smem, stream>>>(
        tm_x, tm_w, (uint16_t*)logits, n, E, H, n_pad, x_box_rows, w_box_rows, status, r);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}
}  // namespace

int launch_gate_logits(const CUtensorMap& tm_x, const CUtensorMap& tm_w, void* logits, int n, int E, int H, int n_pad,
                       int x_box_rows, int w_box_rows, uint32_t* status, cudaStream_t stream) {
    if (n <= 0) return XMOE_OK;
    return launch_gate_t<0>(tm_x, tm_w, logits, n, E, H, n_pad, x_box_rows, w_box_rows, status, RouterArgs{}, stream);
}

// The gate GEMM with the router in its epilogue: `r` as for launch_router_topk (r.logits unused, r.N == n, r.E == E);
// logits may be null.
int launch_gate_route(const CUtensorMap& tm_x, const CUtensorMap& tm_w, void* logits, int n, int E, int H, int n_pad,
                      int x_box_rows, int w_box_rows, uint32_t* status, const RouterArgs& r, cudaStream_t stream) {
    if (n <= 0) return XMOE_OK;
    if (r.n_group > 1 || r.bias != nullptr) {  // the checks of launch_router_topk
        if (r.scoring != 1 || r.lut == nullptr) return XMOE_ERR_SHAPE;
        if (r.n_group < 1 || r.n_group > 32 || E % r.n_group) return XMOE_ERR_SHAPE;
        if (r.n_group > 1 && (E / r.n_group < 2 || r.topk_group < 1 || r.topk_group > r.n_group ||
                              r.topk > r.topk_group * (E / r.n_group)))
            return XMOE_ERR_SHAPE;
        return launch_gate_t<3>(tm_x, tm_w, logits, n, E, H, n_pad, x_box_rows, w_box_rows, status, r, stream);
    }
    return r.scoring == 1 ? launch_gate_t<2>(tm_x, tm_w, logits, n, E, H, n_pad, x_box_rows, w_box_rows, status, r, stream)
                          : launch_gate_t<1>(tm_x, tm_w, logits, n, E, H, n_pad, x_box_rows, w_box_rows, status, r, stream);
}

}  // namespace xmoe
