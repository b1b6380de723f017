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

__device__ __forceinline__ uint32_t ue4m3_ceil(float x) {
    if (!(x > 0.0f)) return 0u;
    if (x >= 448.0f) return 0x7eu;
    const uint32_t bits = __float_as_uint(x);
    int e = int((bits >> 23) & 0xffu) - 120;
    if (e <= 0) {
        const uint32_t m = __float2uint_ru(x * 512.0f);
        return m > 7u ? 7u : m;
    }
    uint32_t m = (bits >> 20) & 7u;
    m += (bits & 0x000fffffu) != 0u;
    if (m == 8u) {
        m = 0u;
        e++;
    }
    if (e >= 15) return m > 6u ? 0x7eu : (0x78u | m);
    return (uint32_t(e) << 3) | m;
}
__device__ __forceinline__ float ue4m3_decode(uint32_t s) {
    const uint32_t e = s >> 3, m = s & 7u;
    if (!e) return float(m) * (1.0f / 512.0f);
    return __uint_as_float(((e + 120u) << 23) | (m << 20));
}
// two bf16 (packed) times a packed bf16 scale, product rounded to bf16, then RN-satfinite E2M1.
__device__ __forceinline__ uint32_t e2m1x2(uint32_t x2, uint32_t scale2) {
    uint32_t q;
    asm("{\n\t"
        ".reg .b32 y;\n\t"
        ".reg .b16 lo, hi;\n\t"
        ".reg .f32 flo, fhi;\n\t"
        ".reg .b8 z;\n\t"
        "mul.rn.bf16x2 y, %1, %2;\n\t"
        "mov.b32 {lo, hi}, y;\n\t"
        "cvt.f32.bf16 flo, lo;\n\t"
        "cvt.f32.bf16 fhi, hi;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 z, fhi, flo;\n\t"
        "cvt.u32.u8 %0, z;\n\t"
        "}"
        : "=r"(q)
        : "r"(x2), "r"(scale2));
    return q;
}

// One thread quantises 16 consecutive K of one token (one block scale, 8 packed bytes);
// a warp covers 512 K. The packet is then stored to each of the token's k_eff rows.
__global__ __launch_bounds__(256) void act_quant_pack_kernel(
    const uint16_t* __restrict__ x, const ActScale* __restrict__ scale, const int32_t* __restrict__ topk_row,
    int N, int H, int k_eff, int idx_stride, uint8_t* __restrict__ xq, uint8_t* __restrict__ sfx, int kb_pad,
    int units_per_token, int nt, const int32_t* __restrict__ n_valid) {
    const float xgs = scale->xgs;
    const uint32_t lane = lane_id();
    if (n_valid) N = min(N, max(*n_valid, 0));
    const size_t total_units = (size_t)N * units_per_token;
    const int h_pad = kb_pad * 64;
    for (size_t unit = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5); unit < total_units;
         unit += (size_t)gridDim.x * 8) {
        const int t = (int)(unit / units_per_token);
        const int h0 = (int)(unit % units_per_token) * 512 + (int)lane * 16;
        // a token none of whose slots got a row (expert id -1 in caller-supplied routing): nothing to store
        bool any_row = false;
        for (int k = 0; k < k_eff; ++k) any_row |= topk_row[(size_t)t * idx_stride + k] >= 0;
        if (!any_row) continue;
        uint32_t w[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (h0 < H) {  // H is a multiple of 16
            const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * H + h0);
            const uint4 a = src[0], b = src[1];
            w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
            w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
        }
        uint32_t mx = 0u;
#pragma unroll
        for (int j = 0; j < 8; ++j) mx = max(mx, max(w[j] & 0x7fffu, (w[j] >> 16) & 0x7fffu));
        uint32_t sbyte = 0u, q_lo = 0u, q_hi = 0u;
        if (mx) {
            sbyte = ue4m3_ceil(bf16_bits_to_f32(mx) * xgs * (1.0f / 6.0f));
            const uint32_t qs = f32_to_bf16_bits(xgs / ue4m3_decode(sbyte));
            const uint32_t qs2 = qs | (qs << 16);
#pragma unroll
            for (int j = 0; j < 4; ++j) q_lo |= e2m1x2(w[j], qs2) << (8 * j);
#pragma unroll
            for (int j = 0; j < 4; ++j) q_hi |= e2m1x2(w[4 + j], qs2) << (8 * j);
        }
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
    act_quant_pack_kernel<<<(int)blocks, 256, 0, stream>>>((const uint16_t*)a.x, a.scale, a.topk_row, a.N, a.H,
                                                           a.k_eff, a.idx_stride, (uint8_t*)a.xq, (uint8_t*)a.sfx,
                                                           a.kb_pad, units_per_token, a.nt, a.n_valid);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

}  // namespace xmoe
