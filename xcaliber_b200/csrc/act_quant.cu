// Activation statistics and NVFP4 activation quantisation.
//
// Arithmetic follows the reference preamble
// (xFused-NVFP4-Kernels/xMoE/xW4A16/sm120a/preamble.cuh):
//   :69-128   tensor-wide amax on bf16 magnitudes, XGS = 2688/amax, XGSINV = bf16(amax/2688)
//   :17-43    round-up UE4M3 block-scale encode and its decode
//   :45-66    bf16x2 * bf16 scale (rounded to bf16) -> RN-satfinite E2M1 pair
//   :567-599  per token, per 16 K: s = ue4m3_ceil(amax16 * XGS / 6), q = e2m1(x * bf16(XGS/dec(s)))
// The layout is new: packed rows [R, H/2] (low nibble = lower K) that TMA can stage
// with a 128-byte swizzle, and scale factors in 512-byte tiles (one per token tile of NT
// rows and 64 K) in exactly the order the tcgen05 scale-factor copy consumes: byte
// (row%32)*16 + (row%NT / 32)*4 + (k16 % 4). A tile always starts at TMEM column 0 of the
// token operand, whatever NT is; for NT < 128 the unused 4-byte groups are never read.
#include "common.cuh"
#include "kernels.h"
#include "nvfp4_quant.cuh"

namespace xmoe {

__global__ __launch_bounds__(256) void act_amax_kernel(const uint4* __restrict__ x, size_t n_vec,
                                                       const uint16_t* __restrict__ tail, int n_tail,
                                                       uint32_t* __restrict__ scratch, ActScale* __restrict__ scale) {
    __shared__ uint32_t warp_max[8];
    // magnitudes of two bf16 at a time (packed unsigned 16-bit max); four independent 16-byte loads
    // in flight per thread
    uint32_t mx2 = 0u;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < n_vec; i += 4 * stride) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = x[i + u * stride];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            mx2 = __vmaxu2(mx2, v[u].x & 0x7fff7fffu);
            mx2 = __vmaxu2(mx2, v[u].y & 0x7fff7fffu);
            mx2 = __vmaxu2(mx2, v[u].z & 0x7fff7fffu);
            mx2 = __vmaxu2(mx2, v[u].w & 0x7fff7fffu);
        }
    }
    for (; i < n_vec; i += stride) {
        const uint4 v = x[i];
        mx2 = __vmaxu2(mx2, v.x & 0x7fff7fffu);
        mx2 = __vmaxu2(mx2, v.y & 0x7fff7fffu);
        mx2 = __vmaxu2(mx2, v.z & 0x7fff7fffu);
        mx2 = __vmaxu2(mx2, v.w & 0x7fff7fffu);
    }
    uint32_t mx = max(mx2 & 0xffffu, mx2 >> 16);
    if (blockIdx.x == 0 && (int)threadIdx.x < n_tail) mx = max(mx, (uint32_t)tail[threadIdx.x] & 0x7fffu);
    mx = __reduce_max_sync(0xffffffffu, mx);
    if (lane_id() == 0) warp_max[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int w = 1; w < 8; ++w) mx = max(mx, warp_max[w]);
        atomicMax(&scratch[0], mx);
        __threadfence();
        const uint32_t ticket = atomicAdd(&scratch[1], 1u);
        if (ticket == gridDim.x - 1) {
            __threadfence();
            const uint32_t m = atomicExch(&scratch[0], 0u);
            scratch[1] = 0u;
            const float amax = bf16_bits_to_f32(m);
            if (m) {
                scale->xgs = 2688.0f / amax;
                scale->xgs_inv = bf16_bits_to_f32(f32_to_bf16_bits(amax * (1.0f / 2688.0f)));
            } else {
                scale->xgs = 0.f;
                scale->xgs_inv = 0.f;
            }
            reinterpret_cast<float*>(scale)[2] = amax;  // third word: the raw maximum
        }
    }
}

// amax (e.g. after a max all-reduce across expert-parallel ranks) -> {XGS, XGSINV, amax}
__global__ void act_scale_from_amax_kernel(const float* __restrict__ amax_in, float* __restrict__ scale) {
    const float amax = *amax_in;
    if (amax > 0.f) {
        scale[0] = 2688.0f / amax;
        scale[1] = bf16_bits_to_f32(f32_to_bf16_bits(amax * (1.0f / 2688.0f)));
    } else {
        scale[0] = 0.f;
        scale[1] = 0.f;
    }
    scale[2] = amax;
}

int launch_act_scale_from_amax(const float* amax, float* scale, cudaStream_t stream) {
    act_scale_from_amax_kernel<<<1, 1, 0, stream>>>(amax, scale);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

// One thread quantises 16 consecutive K of one token (one block scale, 8 packed bytes);
// a warp covers 512 K. The packet is then stored to each of the token's k_eff rows.
// FUSED_AMAX (small batches only): every block first takes the amax of the whole of x itself (a few
// hundred KB, from L2) instead of reading the scale a separate amax kernel left: one launch fewer, same
// bits (the maximum does not depend on the order). Block 0 publishes {XGS, XGSINV, amax} for FF1.
template <bool FUSED_AMAX>
__global__ __launch_bounds__(256) void act_quant_pack_kernel(
    const uint16_t* __restrict__ x, ActScale* __restrict__ scale, const int32_t* __restrict__ topk_row,
    int N, int H, int k_eff, int idx_stride, uint8_t* __restrict__ xq, uint8_t* __restrict__ sfx, int kb_pad,
    int units_per_token, int nt, const int32_t* __restrict__ n_valid) {
    float xgs;
    if (FUSED_AMAX) {
        __shared__ uint32_t warp_max[8];
        const size_t n_vec = (size_t)N * H / 8;  // H is a multiple of 16
        const uint4* xv = reinterpret_cast<const uint4*>(x);
        uint32_t mx2 = 0u;
        for (size_t i = threadIdx.x; i < n_vec; i += blockDim.x) {
            const uint4 v = xv[i];
            mx2 = __vmaxu2(mx2, v.x & 0x7fff7fffu);
            mx2 = __vmaxu2(mx2, v.y & 0x7fff7fffu);
            mx2 = __vmaxu2(mx2, v.z & 0x7fff7fffu);
            mx2 = __vmaxu2(mx2, v.w & 0x7fff7fffu);
        }
        uint32_t mx = max(mx2 & 0xffffu, mx2 >> 16);
        mx = __reduce_max_sync(0xffffffffu, mx);
        if (lane_id() == 0) warp_max[threadIdx.x >> 5] = mx;
        __syncthreads();
#pragma unroll
        for (int w = 0; w < 8; ++w) mx = max(mx, warp_max[w]);
        const float amax = bf16_bits_to_f32(mx);
        xgs = mx ? 2688.0f / amax : 0.f;
        if (blockIdx.x == 0 && threadIdx.x == 0) {  // as act_amax_kernel's last block
            scale->xgs = xgs;
            scale->xgs_inv = mx ? bf16_bits_to_f32(f32_to_bf16_bits(amax * (1.0f / 2688.0f))) : 0.f;
            reinterpret_cast<float*>(scale)[2] = amax;
        }
    } else {
        xgs = scale->xgs;
    }
    const uint32_t lane = lane_id();
    if (n_valid) N = min(N, max(*n_valid, 0));
    const size_t total_units = (size_t)N * units_per_token;
    const int h_pad = kb_pad * 64;
    for (size_t unit = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5); unit < total_units;
         unit += (size_t)gridDim.x * 8) {
        const int t = (int)(unit / units_per_token);
        const int h0 = (int)(unit % units_per_token) * 512 + (int)lane * 16;
        // the token's 16 values are fetched before its row numbers are looked at: the two loads do not depend on
        // each other, and a warp's iterations are a chain of memory latencies
        uint32_t w[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (h0 < H) {  // H is a multiple of 16
            const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * H + h0);
            const uint4 a = __ldg(src), b = __ldg(src + 1);
            w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
            w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
        }
        // a token none of whose slots got a row (expert id -1 in caller-supplied routing): nothing to store
        bool any_row = false;
        for (int k = 0; k < k_eff; ++k) any_row |= topk_row[(size_t)t * idx_stride + k] >= 0;
        if (!any_row) continue;
        uint32_t sbyte, q_lo, q_hi;
        nvfp4_quantise16(w, xgs, sbyte, q_lo, q_hi);
        // four neighbouring lanes hold the four block scales of one K64 block
        uint32_t s4 = sbyte << (8 * (lane & 3u));
        s4 |= __shfl_xor_sync(0xffffffffu, s4, 1);
        s4 |= __shfl_xor_sync(0xffffffffu, s4, 2);
        const int kb = h0 >> 6;
        for (int k = 0; k < k_eff; ++k) {
            const int r = topk_row[(size_t)t * idx_stride + k];
            if (r < 0) continue;
            if (h0 < H) *reinterpret_cast<uint2*>(xq + (size_t)r * (H / 2) + h0 / 2) = make_uint2(q_lo, q_hi);
            if ((lane & 3u) == 0u && h0 < h_pad) {
                const size_t blk = (size_t)(r / nt) * kb_pad + kb;
                *reinterpret_cast<uint32_t*>(sfx + blk * 512 + (r & 31) * 16 + ((r % nt) >> 5) * 4) = s4;
            }
        }
    }
}

// Rows that arrive already quantised (an expert-parallel peer did it with the shared activation
// scale): codes [n, H/2] and block scales [n, H/16] in arrival order -> packed rows and scale tiles.
// One warp per row; the same destinations act_quant_pack_kernel writes.
__global__ __launch_bounds__(256) void act_repack_kernel(const uint8_t* __restrict__ xq_in,
                                                        const uint8_t* __restrict__ sf_in,
                                                        const int32_t* __restrict__ topk_row, int N, int idx_stride, int H,
                                                        uint8_t* __restrict__ xq, uint8_t* __restrict__ sfx, int kb_pad,
                                                        int nt, const int32_t* __restrict__ n_valid) {
    if (n_valid) N = min(N, max(*n_valid, 0));
    const int lane = (int)lane_id();
    const int code_vecs = H / 32;  // 16-byte pieces of one row of codes
    const int groups = H / 64;     // 4 scale bytes per K64 block
    for (int j = blockIdx.x * 8 + (threadIdx.x >> 5); j < N; j += gridDim.x * 8) {
        const int r = topk_row[(size_t)j * idx_stride];
        if (r < 0) continue;
        const uint4* src = reinterpret_cast<const uint4*>(xq_in + (size_t)j * (H / 2));
        uint4* dst = reinterpret_cast<uint4*>(xq + (size_t)r * (H / 2));
        for (int i = lane; i < code_vecs; i += 32) dst[i] = src[i];
        const uint32_t* s_in = reinterpret_cast<const uint32_t*>(sf_in + (size_t)j * (H / 16));
        for (int g = lane; g < kb_pad; g += 32) {
            const uint32_t s4 = g < groups ? s_in[g] : 0u;  // K blocks beyond H are padding: scale 0
            const size_t blk = (size_t)(r / nt) * kb_pad + g;
            *reinterpret_cast<uint32_t*>(sfx + blk * 512 + (r & 31) * 16 + ((r % nt) >> 5) * 4) = s4;
        }
    }
}

int launch_act_repack(const void* xq_in, const void* sf_in, const QuantArgs& a, cudaStream_t stream) {
    if (a.N <= 0) return XMOE_OK;
    if (a.H % 64 || a.k_eff != 1 || (a.nt != 32 && a.nt != 64 && a.nt != 128)) return XMOE_ERR_SHAPE;
    int blocks = (a.N + 7) / 8;
    if (blocks > 148 * 16) blocks = 148 * 16;
    act_repack_kernel<<<blocks, 256, 0, stream>>>((const uint8_t*)xq_in, (const uint8_t*)sf_in, a.topk_row, a.N,
                                                  a.idx_stride, a.H, (uint8_t*)a.xq, (uint8_t*)a.sfx, a.kb_pad, a.nt,
                                                  a.n_valid);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

int launch_act_amax(const AmaxArgs& a, cudaStream_t stream) {
    const size_t n_vec = a.n_elems / 8;
    const int n_tail = (int)(a.n_elems % 8);
    int blocks = (int)((n_vec + 255) / 256);
    blocks = blocks < 1 ? 1 : (blocks > 592 ? 592 : blocks);
    act_amax_kernel<<<blocks, 256, 0, stream>>>((const uint4*)a.x, n_vec, (const uint16_t*)a.x + n_vec * 8, n_tail,
                                                a.scratch, a.scale);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

int launch_act_quant(const QuantArgs& a, cudaStream_t stream) {
    if (a.N <= 0) return XMOE_OK;
    if (a.H % 16 || (a.nt != 32 && a.nt != 64 && a.nt != 128)) return XMOE_ERR_SHAPE;
    const int units_per_token = (a.kb_pad * 64 + 511) / 512;
    const size_t total = (size_t)a.N * units_per_token;
    size_t blocks = (total + 7) / 8;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (a.fused_amax)
        act_quant_pack_kernel<true><<<(int)blocks, 256, 0, stream>>>(
            (const uint16_t*)a.x, const_cast<ActScale*>(a.scale), a.topk_row, a.N, a.H, a.k_eff, a.idx_stride,
            (uint8_t*)a.xq, (uint8_t*)a.sfx, a.kb_pad, units_per_token, a.nt, a.n_valid);
    else
        act_quant_pack_kernel<false><<<(int)blocks, 256, 0, stream>>>(
            (const uint16_t*)a.x, const_cast<ActScale*>(a.scale), a.topk_row, a.N, a.H, a.k_eff, a.idx_stride,
            (uint8_t*)a.xq, (uint8_t*)a.sfx, a.kb_pad, units_per_token, a.nt, a.n_valid);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

}  // namespace xmoe
