// NVFP4 activation quantisation, the arithmetic shared by the local quantise-and-pack kernel and
// the expert-parallel dispatch that quantises on the sending GPU. Same operations, in the same
// order, as the reference's moe_ue4m3_ceil / moe_ue4m3_f32 / moe_e2m1x2_bf16x2 and its packing loop
// (sm120a/preamble.cuh:17-66, 567-599): block scale = round-up UE4M3 of amax * XGS / 6, values
// multiplied by bf16(XGS / decoded scale) in bf16, then round-to-nearest saturating E2M1.
#pragma once

#include "common.cuh"

namespace xmoe {

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
