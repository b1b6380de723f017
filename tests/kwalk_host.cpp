// Host build of the K-walk scheduler (xcaliber_b200/csrc/k_walk.h) for tests/test_abi_cpu.py: compiled with g++,
// no CUDA. Fills out[6 * i ..] = {tile, ks0, ks1, it0, first_helper, finishes} for the i-th segment CTA `cta` walks.
#include "../xcaliber_b200/csrc/k_walk.h"

extern "C" int kwalk_segments(int total_tiles, int k_walk, int grid, int cta, int use_split, int* out, int cap) {
    xmoe::KWalk w;
    w.init(total_tiles, k_walk, grid, cta, use_split != 0);
    for (int i = 0; i < w.n_seg && i < cap; ++i) {
        const xmoe::KSegment g = w.seg(i, cta);
        out[6 * i + 0] = g.tile;
        out[6 * i + 1] = g.ks0;
        out[6 * i + 2] = g.ks1;
        out[6 * i + 3] = g.it0;
        out[6 * i + 4] = g.first_helper;
        out[6 * i + 5] = g.finishes ? 1 : 0;
    }
    return w.n_seg;
}
