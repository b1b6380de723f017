// NVFP4 activation quantisation, the arithmetic shared by the local quantise-and-pack kernel and
// the expert-parallel dispatch that quantises on the sending GPU. The results are, bit for bit,
// those of the reference's quantiser (sm120a/preamble.cuh:17-66, 567-599): block scale = UE4M3 of
// amax * XGS / 6 rounded UP, values multiplied by bf16(XGS / decoded scale) with the product
// rounded to bf16, then round-to-nearest-even saturating E2M1. The formulation is this library's:
// the UE4M3 code is read off the fp32 bit pattern (a UE4M3 normal is an fp32 with the low 20
// mantissa bits dropped and the exponent re-biased by 120, so code = (bits >> 20) - 960), and the
// E2M1 conversion goes through the cuda_fp4.h conversion intrinsic.
#pragma once

#include <cuda_fp4.h>

#include "common.cuh"

namespace xmoe {

constexpr uint32_t kUe4m3Rebias = 120u << 3;  // fp32 exponent 127 against UE4M3 bias 7, in units of 1/8 octave
constexpr uint32_t kUe4m3Max = 0x7eu;         // 448

// Smallest UE4M3 value >= x (x finite, fp32), saturating at 448. Below the normal range (x < 2^-6) the
// code counts 1/512 steps and stops at 7, the largest subnormal.
__device__ __forceinline__ uint32_t ue4m3_ceil(float x) {
    if (!(x > 0.0f)) return 0u;
    const uint32_t bits = __float_as_uint(x);
    if (bits < (121u << 23)) return min(7u, (uint32_t)ceilf(x * 512.0f));
    // adding the dropped bits' all-ones pattern before the shift rounds the 3-bit mantissa up and
    // carries into the exponent on its own
    return min(((bits + 0x000fffffu) >> 20) - kUe4m3Rebias, kUe4m3Max);
}
__device__ __forceinline__ float ue4m3_decode(uint32_t s) {
    return s < 8u ? (float)s * 0x1p-9f : __uint_as_float((s + kUe4m3Rebias) << 20);
}
// Two packed bf16 values times a packed bf16 scale -> one byte of two E2M1 codes (low nibble = the low
// half). The product is rounded to bf16 first, as the reference does with mul.rn.bf16x2.
__device__ __forceinline__ uint32_t e2m1x2(uint32_t x2, uint32_t scale2) {
    const __nv_bfloat162 prod = __hmul2(reinterpret_cast<const __nv_bfloat162&>(x2),
                                        reinterpret_cast<const __nv_bfloat162&>(scale2));
    return (uint32_t)__nv_cvt_float2_to_fp4x2(__bfloat1622float2(prod), __NV_E2M1, cudaRoundNearest);
}

// 16 consecutive bf16 values (8 packed words) of one token -> block-scale byte and 8 bytes of E2M1
// codes (low nibble = lower K). xgs = 2688 / amax of the whole activation tensor.
__device__ __forceinline__ void nvfp4_quantise16(const uint32_t (&w)[8], float xgs, uint32_t& sbyte, uint32_t& q_lo,
                                                 uint32_t& q_hi) {
    uint32_t mx = 0u;
#pragma unroll
    for (int j = 0; j < 8; ++j) mx = max(mx, max(w[j] & 0x7fffu, (w[j] >> 16) & 0x7fffu));
    sbyte = 0u;
    q_lo = 0u;
    q_hi = 0u;
    if (mx) {
        sbyte = ue4m3_ceil(bf16_bits_to_f32(mx) * xgs * (1.0f / 6.0f));
        const uint32_t qs = f32_to_bf16_bits(xgs / ue4m3_decode(sbyte));
        const uint32_t qs2 = qs | (qs << 16);
#pragma unroll
        for (int j = 0; j < 4; ++j) q_lo |= e2m1x2(w[j], qs2) << (8 * j);
#pragma unroll
        for (int j = 0; j < 4; ++j) q_hi |= e2m1x2(w[4 + j], qs2) << (8 * j);
    }
}

}  // namespace xmoe
