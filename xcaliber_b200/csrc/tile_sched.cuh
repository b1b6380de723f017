// Device-side tile list for the grouped GEMMs, and the gated activation shared by the FF1
// epilogues. A work item is (expert, weight tile, token tile); the list is never written to
// memory: every CTA rebuilds the per-expert prefix of tile counts from the expert histogram
// and decodes item numbers with a binary search.
#pragma once

#include "common.cuh"
#include "k_walk.h"

namespace xmoe {

struct TileInfo {
    int e, wt, nt_idx, count, row0;  // expert, weight-tile index, token-tile index, expert rows, first packed row
};

// prefix[e] = number of tiles of experts < e (one warp, 32 experts per step, running carry).
__device__ __forceinline__ void tile_prefix_build(int* prefix, const int32_t* counts, int e_tot, int w_tiles,
                                                  int token_tile) {
    const int lane = threadIdx.x & 31;
    int carry = 0;
    for (int base = 0; base < e_tot; base += 32) {
        const int e = base + lane;
        const int v = e < e_tot ? ((counts[e] + token_tile - 1) / token_tile) * w_tiles : 0;
        int incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += o;
        }
        if (e < e_tot) prefix[e] = carry + incl - v;
        carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) prefix[e_tot] = carry;
}

// Token tiles are innermost, so the CTAs of one wave work on the same weight tile and share
// it through L2.
__device__ __forceinline__ TileInfo tile_decode(int item, const int* prefix, const int32_t* counts,
                                                const int32_t* offsets, int e_tot, int token_tile) {
    int lo = 0, hi = e_tot;  // largest e with prefix[e] <= item
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (prefix[mid] <= item) lo = mid; else hi = mid;
    }
    TileInfo t;
    t.e = lo;
    const int local = item - prefix[lo];
    t.count = counts[lo];
    const int n_tiles = (t.count + token_tile - 1) / token_tile;
    t.wt = local / n_tiles;
    t.nt_idx = local % n_tiles;
    t.row0 = offsets[lo] + t.nt_idx * token_tile;
    return t;
}

// The one GLU epilogue all FF1 kernels use (activation 0: silu(g)*u; 1: clamped SwiGLU
// (min(g,limit) * sigmoid(alpha*g)) * (clamp(u)+1); 2: tanh-GELU(g)*u; fp32 with the approximate ex2 /
// rcp units, like the reference epilogue, xR64FF1.cu:356-386). g_acc / u_acc are the raw fp32 accumulators, sg the
// gate scale (weight_global_scale * XGSINV), su_w the up scale times the routing weight, w the
// routing weight (needed on its own only where the activation adds a constant to u). Every
// operation is an explicit round-to-nearest intrinsic so that the compiler cannot contract or
// reorder differently in different kernels: the decode and prefill variants, and therefore the
// single-GPU and expert-parallel paths, produce bit-identical rows.
__device__ __forceinline__ float glu_apply(int act, float g_acc, float u_acc, float sg, float su_w, float alpha,
                                           float limit, float w) {
    float g = __fmul_rn(g_acc, sg);
    float u_w = __fmul_rn(u_acc, su_w);
    if (act == 1) {  // clamped SwiGLU: min(g,limit) * sigmoid(alpha*g) * (clamp(u,-limit,limit) + 1) * w
        g = fminf(g, limit);
        const float lw = __fmul_rn(limit, fabsf(w));
        u_w = fminf(fmaxf(u_w, -lw), lw);
        const float e = ex2_approx(__fmul_rn(__fmul_rn(g, alpha), -1.4426950408889634f));
        const float sgm = rcp_approx(__fadd_rn(1.0f, e));
        return __fmul_rn(__fmul_rn(g, sgm), __fadd_rn(u_w, w));
    }
    if (act == 2) {  // tanh-GELU(g) * u * w
        const float g3 = __fmul_rn(__fmul_rn(g, g), g);
        const float inner = __fmul_rn(0.7978845608028654f, __fmaf_rn(0.044715f, g3, g));
        const float e = ex2_approx(__fmul_rn(inner, 2.0f * 1.4426950408889634f));
        const float t = __fmaf_rn(-2.0f, rcp_approx(__fadd_rn(1.0f, e)), 1.0f);
        return __fmul_rn(__fmul_rn(__fmul_rn(0.5f, g), __fadd_rn(1.0f, t)), u_w);
    }
    const float e = ex2_approx(__fmul_rn(g, -1.4426950408889634f));  // silu(g) * u * w
    return __fmul_rn(__fmul_rn(g, u_w), rcp_approx(__fadd_rn(1.0f, e)));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

}  // namespace xmoe
