// Which tiles, and which K units of them, a CTA of a persistent grouped-GEMM kernel works on. Plain C++ (no CUDA
// types) so that the host can run the same code: tests/test_abi_cpu.py walks it exhaustively on the CPU.
#pragma once

#if defined(__CUDACC__)
#define XMOE_HD __host__ __device__ __forceinline__
#else
#define XMOE_HD inline
#endif

namespace xmoe {

// Persistent kernels walk the tile list with a stride. Striding by the grid size leaves the
// last round mostly idle when the tile count is a little above a multiple of it (896 tiles on 148
// CTAs: six full rounds and one of 8 tiles). With the same number of rounds, the smallest stride
// that covers the list spreads the tiles evenly (896 -> 7 rounds of 128): in a bandwidth-bound
// kernel every round then moves data at full rate. CTAs beyond the stride have no tiles.
XMOE_HD int balanced_stride(int total_tiles, int grid) {
    if (total_tiles <= 0) return grid;
    const int rounds = (total_tiles + grid - 1) / grid;
    return (total_tiles + rounds - 1) / rounds;
}

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

    XMOE_HD void init(int total_tiles, int k_walk_, int grid, int cta, bool use_split) {
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
    XMOE_HD KSegment seg(int i, int cta) const {
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

}  // namespace xmoe
