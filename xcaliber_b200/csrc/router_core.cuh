// Per-token routing routines (one warp per token), shared by the router kernels (router.cu, logits from HBM) and
// by the gate GEMM that routes in its own epilogue (gate.cu, logits from shared memory): the same code, so the
// same bits.
//
// Flat top-k: semantics follow the reference router xFused-NVFP4-Kernels/xMoE/xW4A16/sm120a/topk.cuh:25-142
// (selection on the ordered bf16 bit pattern, ties to the lower expert id, slots in descending logit order,
// weights normalised over the selected k).
#pragma once
#include "common.cuh"

namespace xmoe {

// One token, one warp: `row` = the token's E <= 32 * J bf16 logits (global or shared memory), lane l owns experts l + 32*j;
// every composite key lives in a register, so the logits are read exactly once. Writes slots [0, topk) of
// topk_idx / topk_w at token * idx_stride.
// J = slots per lane (ceil(E / 32) rounded up to 1, 2, 4, 8 or 32): the loops over a lane's experts are fully unrolled,
// and a 128-expert router should not walk 32 slots of which 28 are empty.
template <bool SIGMOID, int J>
__device__ __forceinline__ void route_token_flat(const uint16_t* row, uint32_t lane, uint32_t token,
                                                 const uint16_t* __restrict__ expert_scale,
                                                 int32_t* __restrict__ topk_idx, uint16_t* __restrict__ topk_w, int E,
                                                 int topk, int idx_stride, float routed_scale, int renorm) {
    uint32_t keys[J];
#pragma unroll
    for (int j = 0; j < J; ++j) {
        const uint32_t e = lane + 32u * j;
        uint32_t key = 0u;
        if (e < (uint32_t)E) {
            const uint32_t raw = row[e];
            // monotone map of the bf16 bits to unsigned: negatives flip all bits,
            // non-negatives set the sign bit (+0 ranks above -0).
            const uint32_t ord = raw ^ ((0u - (raw >> 15)) | 0x8000u);
            key = (ord << 16) | (0xffffu - e);
        }
        keys[j] = key;
    }

    // Without renormalisation the softmax denominator runs over all E experts.
    float all_sum = 0.f;
    if (!SIGMOID && !renorm) {
        uint32_t best = 0u;
#pragma unroll
        for (int j = 0; j < J; ++j) best = max(best, keys[j]);
        const uint32_t o1 = __reduce_max_sync(0xffffffffu, best) >> 16;
        const float x1 = bf16_bits_to_f32((o1 & 0x8000u) ? (o1 & 0x7fffu) : (~o1 & 0xffffu));
#pragma unroll
        for (int j = 0; j < J; ++j) {
            if (lane + 32u * j < (uint32_t)E) {
                const uint32_t o = keys[j] >> 16;
                const float xe = bf16_bits_to_f32((o & 0x8000u) ? (o & 0x7fffu) : (~o & 0xffffu));
                all_sum += ex2_approx((xe - x1) * 1.4426950408889634f);
            }
        }
#pragma unroll
        for (int d = 16; d; d >>= 1) all_sum += __shfl_xor_sync(0xffffffffu, all_sum, d);
    }

    uint32_t selected = 0u;
    for (int r = 0; r < topk; ++r) {
        uint32_t best = 0u;
#pragma unroll
        for (int j = 0; j < J; ++j) best = max(best, keys[j]);
        const uint32_t winner = __reduce_max_sync(0xffffffffu, best);
        const uint32_t e = 0xffffu - (winner & 0xffffu);
        if ((e & 31u) == lane) {
#pragma unroll
            for (int j = 0; j < J; ++j)
                if ((uint32_t)j == (e >> 5)) keys[j] = 0u;
        }
        if (lane == (uint32_t)r) selected = winner;
    }

    float x = 0.f;
    uint32_t expert = 0u;
    if (lane < (uint32_t)topk) {
        expert = 0xffffu - (selected & 0xffffu);
        const uint32_t ord = selected >> 16;
        const uint32_t raw = (ord & 0x8000u) ? (ord & 0x7fffu) : (~ord & 0xffffu);
        x = bf16_bits_to_f32(raw);
    }
    const float top1 = __shfl_sync(0xffffffffu, x, 0);
    float w = 0.f;
    if (lane < (uint32_t)topk) {
        if (SIGMOID) {
            w = rcp_approx(1.0f + ex2_approx(-x * 1.4426950408889634f));
        } else {
            w = ex2_approx((x - top1) * 1.4426950408889634f);
        }
    }
    float denom = w;
#pragma unroll
    for (int d = 16; d; d >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, d);
    if (lane < (uint32_t)topk) {
        if (renorm) w *= rcp_approx(denom);
        else if (!SIGMOID) w *= rcp_approx(all_sum);
        w *= routed_scale;
        if (expert_scale) w *= bf16_bits_to_f32(expert_scale[expert]);
        topk_idx[(size_t)token * idx_stride + lane] = (int32_t)expert;
        topk_w[(size_t)token * idx_stride + lane] = (uint16_t)f32_to_bf16_bits(w);
    }
}

// ------------------------------------------------------------------------------------
// Group-limited sigmoid routing with a selection bias (DeepSeek-V3 style). Not in the
// reference (its sigmoid mode is flat): score = lut[bf16 logit] (a 65536-entry fp32
// table of sigmoid, so selection is reproducible bit for bit on any machine), choice
// score = score + bias[e]; a group's score is the sum of its two best choice scores;
// the best `topk_group` groups stay; top-k over the choice scores of the remaining
// experts; ties always go to the lower index. Weights are the unbiased scores of the
// winners, normalised over k, times routed_scale.
// ------------------------------------------------------------------------------------
// Largest 64-bit key of the warp: two 32-bit warp reductions (the largest high word, then the largest low word
// among the lanes that hold it) instead of five rounds of 64-bit shuffles.
__device__ __forceinline__ uint64_t warp_max_u64(uint64_t v) {
    const uint32_t hi = (uint32_t)(v >> 32), lo = (uint32_t)v;
    const uint32_t best_hi = __reduce_max_sync(0xffffffffu, hi);
    const uint32_t best_lo = __reduce_max_sync(0xffffffffu, hi == best_hi ? lo : 0u);
    return ((uint64_t)best_hi << 32) | best_lo;
}
__device__ __forceinline__ uint32_t ordered_f32(float f) {
    const uint32_t b = __float_as_uint(f);
    return b ^ ((0u - (b >> 31)) | 0x80000000u);
}
__device__ __forceinline__ float unordered_f32(uint32_t o) {
    const uint32_t b = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
    return __uint_as_float(b);
}

// One token, one warp, group-limited selection. J = ceil(E / 32) slots per lane, as a template parameter: the
// loops over a lane's experts are fully unrolled (keys live in registers), and the DeepSeek-V3 shape (E = 256)
// needs 8 of them, not 32.
template <int J>
__device__ __forceinline__ void route_token_grouped(const uint16_t* row, uint32_t lane, uint32_t token,
                                                    const float* __restrict__ lut, const float* __restrict__ bias,
                                                    const uint16_t* __restrict__ expert_scale,
                                                    int32_t* __restrict__ topk_idx, uint16_t* __restrict__ topk_w, int E,
                                                    int topk, int idx_stride, int n_group, int topk_group,
                                                    float routed_scale, int renorm) {
    const uint32_t gs = (uint32_t)E / (uint32_t)n_group;

    // key = {ordered choice score, ~expert}; 0 = absent / dead. gid = the expert's group (one division per slot,
    // not one per slot and group)
    uint64_t keys[J];
    float score[J];
    int gid[J];
#pragma unroll
    for (int j = 0; j < J; ++j) {
        const uint32_t e = lane + 32u * j;
        keys[j] = 0ull;
        score[j] = 0.f;
        gid[j] = e < (uint32_t)E ? (int)(e / gs) : -1;
        if (e < (uint32_t)E) {
            const float s = lut[row[e]];
            score[j] = s;
            const float c = bias ? __fadd_rn(s, bias[e]) : s;
            keys[j] = ((uint64_t)ordered_f32(c) << 32) | (uint64_t)(0xffffffffu - e);
        }
    }

    // group scores -> allowed-group mask (n_group <= 32)
    uint32_t allowed = 0xffffffffu;
    if (n_group > 1) {
        float gscore = 0.f;  // lane g keeps group g's score
        for (int g = 0; g < n_group; ++g) {
            uint64_t b1 = 0ull;
#pragma unroll
            for (int j = 0; j < J; ++j)
                if (gid[j] == g) b1 = keys[j] > b1 ? keys[j] : b1;
            const uint64_t w1 = warp_max_u64(b1);
            uint64_t b2 = 0ull;
#pragma unroll
            for (int j = 0; j < J; ++j)
                if (gid[j] == g && keys[j] != w1) b2 = keys[j] > b2 ? keys[j] : b2;
            const uint64_t w2 = warp_max_u64(b2);
            const float sum = __fadd_rn(unordered_f32((uint32_t)(w1 >> 32)), unordered_f32((uint32_t)(w2 >> 32)));
            if (lane == (uint32_t)g) gscore = sum;
        }
        allowed = 0u;
        uint64_t gkey = lane < (uint32_t)n_group
                            ? (((uint64_t)ordered_f32(gscore) << 32) | (uint64_t)(0xffffffffu - lane))
                            : 0ull;
        for (int r = 0; r < topk_group; ++r) {
            const uint64_t wg = warp_max_u64(gkey);
            const uint32_t g = 0xffffffffu - (uint32_t)wg;
            allowed |= 1u << g;
            if (lane == g) gkey = 0ull;
        }
#pragma unroll
        for (int j = 0; j < J; ++j)
            if (gid[j] >= 0 && !((allowed >> gid[j]) & 1u)) keys[j] = 0ull;
    }

    float my_score = 0.f;
    uint32_t my_expert = 0u;
    for (int r = 0; r < topk; ++r) {
        uint64_t best = 0ull;
#pragma unroll
        for (int j = 0; j < J; ++j) best = keys[j] > best ? keys[j] : best;
        const uint64_t winner = warp_max_u64(best);
        const uint32_t e = 0xffffffffu - (uint32_t)winner;
        float s = 0.f;
        if ((e & 31u) == lane) {
#pragma unroll
            for (int j = 0; j < J; ++j)
                if ((uint32_t)j == (e >> 5)) {
                    keys[j] = 0ull;
                    s = score[j];
                }
        }
        s = __shfl_sync(0xffffffffu, s, e & 31u);
        if (lane == (uint32_t)r) {
            my_score = s;
            my_expert = e;
        }
    }
    // fixed-order sum over the k slots (slot 0 first) so that the host restatement
    // can reproduce it with plain fp32 adds.
    float denom = 0.f;
    for (int r = 0; r < topk; ++r) denom = __fadd_rn(denom, __shfl_sync(0xffffffffu, my_score, r));
    if (lane < (uint32_t)topk) {
        float w = my_score;
        if (renorm) w = __fdiv_rn(w, denom);
        w = __fmul_rn(w, routed_scale);
        if (expert_scale) w *= bf16_bits_to_f32(expert_scale[my_expert]);
        topk_idx[(size_t)token * idx_stride + lane] = (int32_t)my_expert;
        topk_w[(size_t)token * idx_stride + lane] = (uint16_t)f32_to_bf16_bits(w);
    }
}

}  // namespace xmoe
