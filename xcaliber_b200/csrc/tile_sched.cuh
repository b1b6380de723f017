// Device-side tile list for the grouped GEMMs, and the gated activation shared by the FF1
// epilogues. A work item is (expert, weight tile, token tile); the list is never written to
// memory: every CTA rebuilds the per-expert prefix of tile counts from the expert histogram
// and decodes item numbers with a binary search.
#pragma once

#include "common.cuh"

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

__device__ __forceinline__ int balanced_stride(int total_tiles, int grid);

// ---- tiles cut along K ("stream-K") ----------------------------------------------------------------
// With few tiles per SM (decode: 256 tiles on 148 SMs) whole-tile scheduling leaves SMs idle for a whole
// round. Here the K units of all tiles, tile after tile, form one line of total_tiles * k_walk units and CTA
// c takes the units [c * span, (c + 1) * span): every CTA streams the same number of weight bytes. A CTA's
// share is a list of segments (tile, K units [ks0, ks1)); at most its last one (in tile order) stops short
// of the tile's end. Such a NON-FINAL segment only produces a partial sum, which the CTA leaves in its
// scratch slot for the CTA that finishes the tile; it is processed FIRST, so that partial sums never wait
// for anything and the CTAs that finish tiles (they wait, bounded, for the helpers' flags) cannot deadlock.
// The finishing CTA adds the helpers' partial sums in K order, then its own: results are deterministic
// for a given tile list and grid. Spans are multiples of 4 K units so that a segment never starts inside
// a two-unit weight stage.
struct KSegment {
    int tile;          // index into the tile list (tile_decode)
    int ks0, ks1;      // K units [ks0, ks1) of the tile
    int it0;           // K units this CTA has walked before the segment (ring numbering)
    int first_helper;  // CTAs [first_helper, this CTA) each hold a partial sum of this tile; == this CTA when ks0 == 0
    bool finishes;     // ks1 reaches the tile's end: this CTA stores the tile
};

struct KWalk {
    int n_seg;
    // whole tiles, balanced stride
    int first_tile, tile_stride, k_walk;
    // stream-K
    int split, u0, span, t0, t1, u1;
    bool rotate;  // the last segment in tile order is non-final and not the only one: it is walked first

    __device__ __forceinline__ void init(int total_tiles, int k_walk_, int grid, int cta, bool use_split) {
        k_walk = k_walk_;
        split = use_split ? 1 : 0;
        first_tile = tile_stride = u0 = u1 = span = t0 = t1 = 0;
        rotate = false;
        if (!use_split) {
            tile_stride = balanced_stride(total_tiles, grid);
            first_tile = cta < tile_stride ? cta : total_tiles;
            n_seg = first_tile < total_tiles ? (total_tiles - 1 - first_tile) / tile_stride + 1 : 0;
            return;
        }
        const long long units = (long long)total_tiles * k_walk;
        span = (int)((units + grid - 1) / grid);
        span = (span + 3) & ~3;
        const long long b0 = (long long)cta * span;
        u0 = (int)(b0 < units ? b0 : units);
        u1 = (int)(b0 + span < units ? b0 + span : units);
        n_seg = 0;
        rotate = false;
        if (u0 >= u1) return;
        t0 = u0 / k_walk;
        t1 = (u1 - 1) / k_walk;
        n_seg = t1 - t0 + 1;
        rotate = n_seg > 1 && (u1 - t1 * k_walk) < k_walk;
    }
    // i-th segment in the order this CTA walks them
    __device__ __forceinline__ KSegment seg(int i, int cta) const {
        KSegment g;
        if (!split) {
            g.tile = first_tile + i * tile_stride;
            g.ks0 = 0;
            g.ks1 = k_walk;
            g.it0 = i * k_walk;
            g.first_helper = cta;
            g.finishes = true;
            return g;
        }
        const int last = n_seg - 1;
        const int j = rotate ? (i == 0 ? last : i - 1) : i;  // position in tile order
        g.tile = t0 + j;
        g.ks0 = j == 0 ? u0 - t0 * k_walk : 0;
        g.ks1 = j == last ? u1 - t1 * k_walk : k_walk;
        g.finishes = g.ks1 == k_walk;
        g.first_helper = g.ks0 == 0 ? cta : (int)(((long long)g.tile * k_walk) / span);
        // units walked before: the rotated tail first, then the segments before j in tile order
        int before = 0;
        if (rotate && i > 0) before += u1 - t1 * k_walk;                 // the tail segment, walked first
        if (j > 0 && !(rotate && i == 0)) before += (t0 + j) * k_walk - u0;  // everything from u0 up to this tile
        g.it0 = before;
        return g;
    }
};

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

// Persistent kernels walk the tile list with a stride. Striding by the grid size leaves the
// last round mostly idle when the tile count is a little above a multiple of it (896 tiles on 148
// CTAs: six full rounds and one of 8 tiles). With the same number of rounds, the smallest stride
// that covers the list spreads the tiles evenly (896 -> 7 rounds of 128): in a bandwidth-bound
// kernel every round then moves data at full rate. CTAs beyond the stride have no tiles.
__device__ __forceinline__ int balanced_stride(int total_tiles, int grid) {
    if (total_tiles <= 0) return grid;
    const int rounds = (total_tiles + grid - 1) / grid;
    return (total_tiles + rounds - 1) / rounds;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

}  // namespace xmoe
