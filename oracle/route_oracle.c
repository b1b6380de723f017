/*
 * Plain-C restatement of the integer/bit-level parts of the reference's MoE preamble.
 * TEST INFRASTRUCTURE ONLY: compiled by oracle/build_oracle.py into oracle/liboracle_c.so and
 * called from tests/ to cross-check the numpy oracle on larger inputs. Not linked into, or
 * loaded by, the product library.
 *
 * Reference (paths inside the xCaliber tree, S = xFused-NVFP4-Kernels/xMoE/xW4A16/sm120a):
 *   orc_router_topk     S/topk.cuh:44-93      selection order and tie rule
 *   orc_route_pack      S/benchmarks/benchmark.cu:172-183 (CPU twin of S/preamble.cuh:466-535)
 *   orc_act_scale       S/preamble.cuh:98-128
 *   orc_ue4m3_ceil      S/preamble.cuh:17-36
 *   orc_ue4m3_decode    S/preamble.cuh:38-43
 *   orc_act_quant_row   S/preamble.cuh:45-66, 567-599
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static uint16_t f32_to_bf16_rn(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* Larger logit wins; equal bf16 patterns -> lower expert id; +0 beats -0 (bit order). */
static int logit_before(uint16_t a, int ea, uint16_t b, int eb) {
    int32_t ka = (a & 0x8000u) ? -(int32_t)(a & 0x7fffu) - 1 : (int32_t)a;
    int32_t kb = (b & 0x8000u) ? -(int32_t)(b & 0x7fffu) - 1 : (int32_t)b;
    if (ka != kb) return ka > kb;
    return ea < eb;
}

void orc_router_topk(const uint16_t* logits, int n, int e, int topk, int32_t* idx) {
    for (int t = 0; t < n; ++t) {
        const uint16_t* row = logits + (size_t)t * e;
        uint8_t taken[1024] = {0};
        for (int r = 0; r < topk; ++r) {
            int best = -1;
            for (int j = 0; j < e; ++j) {
                if (taken[j]) continue;
                if (best < 0 || logit_before(row[j], j, row[best], best)) best = j;
            }
            taken[best] = 1;
            idx[(size_t)t * topk + r] = best;
        }
    }
}

/* Reference containers: topk_off u16 [N,k], expert_topk_W u16 [E,NP], expert_token_idx u16 [E,NP+1]. */
void orc_route_pack(const int32_t* idx, const uint16_t* w, int n, int e, int topk, int np, uint16_t* topk_off,
                    uint16_t* expert_topk_w, uint16_t* expert_token_idx) {
    memset(expert_topk_w, 0, (size_t)e * np * sizeof(uint16_t));
    memset(expert_token_idx, 0, (size_t)e * (np + 1) * sizeof(uint16_t));
    for (int t = 0; t < n; ++t) {
        for (int s = 0; s < topk; ++s) {
            const int ex = idx[(size_t)t * topk + s];
            uint16_t* cnt = &expert_token_idx[(size_t)ex * (np + 1)];
            const uint16_t p = *cnt;
            topk_off[(size_t)t * topk + s] = p;
            expert_topk_w[(size_t)ex * np + p] = w[(size_t)t * topk + s];
            cnt[1 + p] = (uint16_t)t;
            *cnt = (uint16_t)(p + 1);
        }
    }
}

void orc_act_scale(const uint16_t* x, size_t n, float* xgs, float* xgs_inv) {
    uint16_t m = 0;
    for (size_t i = 0; i < n; ++i) {
        const uint16_t a = x[i] & 0x7fffu;
        if (a > m) m = a;
    }
    if (!m) {
        *xgs = 0.f;
        *xgs_inv = 0.f;
        return;
    }
    const float amax = bf16_to_f32(m);
    *xgs = 2688.0f / amax;
    *xgs_inv = bf16_to_f32(f32_to_bf16_rn(amax * (1.0f / 2688.0f)));
}

/* Smallest UE4M3 value >= x (3 mantissa bits, bias 7), except below 2^-6 where the code is
 * min(ceil(512 x), 7); saturates at 448 (0x7e). */
uint32_t orc_ue4m3_ceil(float x) {
    if (!(x > 0.0f)) return 0u;
    if (x >= 448.0f) return 0x7eu;
    int ex;
    const float mant = frexpf(x, &ex); /* x = mant * 2^ex, mant in [0.5, 1) */
    const int e = ex - 1 + 7;          /* biased exponent of the 1.m form */
    if (e <= 0) {
        const float c = ceilf(x * 512.0f);
        return c > 7.0f ? 7u : (uint32_t)c;
    }
    int m = (int)ceilf((mant * 2.0f - 1.0f) * 8.0f);
    int eb = e;
    if (m == 8) {
        m = 0;
        eb++;
    }
    if (eb >= 15) return m > 6 ? 0x7eu : (0x78u | (uint32_t)m);
    return ((uint32_t)eb << 3) | (uint32_t)m;
}

float orc_ue4m3_decode(uint32_t s) {
    const uint32_t e = s >> 3, m = s & 7u;
    if (!e) return (float)m / 512.0f;
    return ldexpf(1.0f + (float)m / 8.0f, (int)e - 7);
}

/* Nearest E2M1 (ties to even mantissa bit), saturating; sign bit from the input. */
static uint8_t e2m1_rn(float v) {
    static const float mid[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
    const float a = fabsf(v);
    uint8_t code = 0;
    for (int i = 0; i < 7; ++i) {
        /* the midpoint above an even code stays down, above an odd code goes up */
        if ((i & 1) ? (a >= mid[i]) : (a > mid[i])) code = (uint8_t)(i + 1);
    }
    return (uint8_t)(code | (signbit(v) ? 8u : 0u));
}

/* One token row: codes[H] (one nibble per element), sf[H/16]. */
void orc_act_quant_row(const uint16_t* x, int h, float xgs, uint8_t* codes, uint8_t* sf) {
    for (int b = 0; b < h / 16; ++b) {
        uint16_t m = 0;
        for (int j = 0; j < 16; ++j) {
            const uint16_t a = x[b * 16 + j] & 0x7fffu;
            if (a > m) m = a;
        }
        if (!m) {
            sf[b] = 0;
            memset(codes + b * 16, 0, 16);
            continue;
        }
        const uint32_t s = orc_ue4m3_ceil(bf16_to_f32(m) * xgs * (1.0f / 6.0f));
        sf[b] = (uint8_t)s;
        const float qs = bf16_to_f32(f32_to_bf16_rn(xgs / orc_ue4m3_decode(s)));
        for (int j = 0; j < 16; ++j) {
            const float prod = bf16_to_f32(f32_to_bf16_rn(bf16_to_f32(x[b * 16 + j]) * qs));
            codes[b * 16 + j] = e2m1_rn(prod);
        }
    }
}
