// Memory-bound helpers around the two grouped GEMMs: the top-k combine back to token
// order, the optional activation top-k on the FF1 output, and the load-time weight
// preparation (scale-factor reorder for the block-scaled MMA, int4 repacks for FF2).
#include "common.cuh"
#include "kernels.h"

namespace xmoe {

// ------------------------------------------------------------------------------------
// Combine: y[t, :] = sum_k rows[topk_row[t, k], :] in fp32, slot 0 first, one bf16 round.
// The routing weight was already applied after SwiGLU (reference operator identity,
// co-design.md:75-90), so the sum is unweighted. Fixed order => run-to-run deterministic,
// unlike the reference's bulk bf16 reduce-adds (xR64FF2.cu tail).
// ------------------------------------------------------------------------------------
__global__ __launch_bounds__(256) void combine_kernel(const uint4* __restrict__ rows,
                                                      const int32_t* __restrict__ topk_row, uint4* __restrict__ y,
                                                      int N, int hv, int k_eff, int idx_stride) {
    const size_t total = (size_t)N * hv;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / hv), c = (int)(i % hv);
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int k = 0; k < k_eff; ++k) {
            const int r = topk_row[(size_t)t * idx_stride + k];
            if (r < 0) continue;
            const uint4 v = rows[(size_t)r * hv + c];
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                acc[2 * j] += bf16_bits_to_f32(w[j] & 0xffffu);
                acc[2 * j + 1] += bf16_bits_to_f32(w[j] >> 16);
            }
        }
        uint4 o;
        o.x = f32_to_bf16_bits(acc[0]) | (f32_to_bf16_bits(acc[1]) << 16);
        o.y = f32_to_bf16_bits(acc[2]) | (f32_to_bf16_bits(acc[3]) << 16);
        o.z = f32_to_bf16_bits(acc[4]) | (f32_to_bf16_bits(acc[5]) << 16);
        o.w = f32_to_bf16_bits(acc[6]) | (f32_to_bf16_bits(acc[7]) << 16);
        y[i] = o;
    }
}

// Destination table for FF2 rows that go straight to a token-major buffer rows_out [N * k_eff, H]: packed row
// topk_row[t, s] -> byte address of row t * k_eff + s (slots without a row are skipped; row_dst is zeroed first,
// so padding rows keep "nowhere").
__global__ void scatter_row_dst_kernel(const int32_t* __restrict__ topk_row, int n_slots, size_t row_bytes,
                                       unsigned long long base, unsigned long long* __restrict__ row_dst) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_slots; i += gridDim.x * blockDim.x) {
        const int r = topk_row[i];
        if (r >= 0) row_dst[r] = base + (unsigned long long)i * row_bytes;
    }
}

int launch_scatter_row_dst(const int32_t* topk_row, int n_slots, int hidden, void* rows_out, unsigned long long* row_dst,
                           cudaStream_t stream) {
    if (n_slots <= 0) return XMOE_OK;
    int blocks = (n_slots + 255) / 256;
    if (blocks > 148 * 4) blocks = 148 * 4;
    scatter_row_dst_kernel<<<blocks, 256, 0, stream>>>(topk_row, n_slots, (size_t)hidden * 2,
                                                       (unsigned long long)(uintptr_t)rows_out, row_dst);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

int launch_combine(const CombineArgs& a, cudaStream_t stream) {
    if (a.N <= 0) return XMOE_OK;
    if (a.H % 8) return XMOE_ERR_SHAPE;
    const int hv = a.H / 8;
    size_t blocks = ((size_t)a.N * hv + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    combine_kernel<<<(int)blocks, 256, 0, stream>>>((const uint4*)a.rows, a.topk_row, (uint4*)a.y, a.N, hv, a.k_eff,
                                                    a.idx_stride);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

// ------------------------------------------------------------------------------------
// Activation top-k (no counterpart in the reference; rule: per packed row keep the
// `keep` entries of largest |y| as bf16 magnitudes, ties to the lower index, zero the
// rest). One CTA per row: two-level radix select on the 15-bit magnitude, then an
// index-ordered pass that hands the remaining quota to the first ties.
// ------------------------------------------------------------------------------------
constexpr int kTopkThreads = 256;
constexpr int kTopkMaxExperts = 1024 + 8;

__global__ __launch_bounds__(kTopkThreads) void act_topk_general_kernel(uint16_t* __restrict__ yact,
                                                                const int32_t* __restrict__ counts,
                                                                const int32_t* __restrict__ offsets, int e_tot, int I,
                                                                int keep) {
    __shared__ int hist[256];
    __shared__ int sel_bucket, sel_above, thr_value, need_equal;
    __shared__ int seg_eq[kTopkThreads];
    // which packed row is this? rows of expert e are [offsets[e], offsets[e] + counts[e])
    const int r = blockIdx.x;
    int lo = 0, hi = e_tot;  // largest e with offsets[e] <= r
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (offsets[mid] <= r) lo = mid; else hi = mid;
    }
    if (r >= offsets[e_tot] || r - offsets[lo] >= counts[lo]) return;
    uint16_t* row = yact + (size_t)r * I;

    // level 1: high 8 bits of the magnitude
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < I; i += blockDim.x) atomicAdd(&hist[(row[i] & 0x7fffu) >> 7], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int above = 0, b = 255;
        for (; b > 0; --b) {
            if (above + hist[b] >= keep) break;
            above += hist[b];
        }
        sel_bucket = b;
        sel_above = above;
    }
    __syncthreads();
    const int bucket = sel_bucket;
    const int above1 = sel_above;
    __syncthreads();
    // level 2: low 7 bits inside the selected bucket
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < I; i += blockDim.x) {
        const int m = row[i] & 0x7fffu;
        if ((m >> 7) == bucket) atomicAdd(&hist[m & 127], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int above = above1, b = 127;
        for (; b > 0; --b) {
            if (above + hist[b] >= keep) break;
            above += hist[b];
        }
        thr_value = (bucket << 7) | b;
        need_equal = keep - above;  // how many entries equal to the threshold survive
    }
    __syncthreads();
    const int thr = thr_value;
    // index-ordered pass: thread i owns the contiguous segment [i*seg, (i+1)*seg)
    const int seg = (I + blockDim.x - 1) / blockDim.x;
    const int s0 = threadIdx.x * seg, s1 = min(I, s0 + seg);
    int eq = 0;
    for (int i = s0; i < s1; ++i) eq += (row[i] & 0x7fffu) == thr;
    seg_eq[threadIdx.x] = eq;
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int i = 0; i < (int)blockDim.x; ++i) {
            const int v = seg_eq[i];
            seg_eq[i] = run;
            run += v;
        }
    }
    __syncthreads();
    int quota = need_equal - seg_eq[threadIdx.x];
    for (int i = s0; i < s1; ++i) {
        const int m = row[i] & 0x7fffu;
        if (m > thr) continue;
        if (m == thr && quota > 0) {
            --quota;
            continue;
        }
        row[i] = 0;
    }
}


// Suffix search over a shared-memory histogram by one warp: the largest bucket b (>= 1, or 0) such
// that the entries in buckets above b number fewer than `keep` while including b reaches it.
// n_bins = 32 * per_lane. Returns through (bucket, above); all lanes get the same values.
template <int PER_LANE>
__device__ __forceinline__ void topk_find_bucket(const int* hist, int keep, int above0, int& bucket, int& above) {
    const int lane = threadIdx.x & 31;
    int mine[PER_LANE], tot = 0;
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
        mine[j] = hist[lane * PER_LANE + j];
        tot += mine[j];
    }
    // inclusive suffix sum over lanes (lane 31 first)
    int suf = tot;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_down_sync(0xffffffffu, suf, d);
        if (lane + d < 32) suf += o;
    }
    // the lane whose range holds the threshold: entries above its range < keep <= entries from its range up
    const int above_lane = above0 + suf - tot;
    const bool has = above_lane < keep && above_lane + tot >= keep;
    const unsigned m = __ballot_sync(0xffffffffu, has);
    int b = 0, ab = above0;
    if (m) {
        const int src = 31 - __clz(m);  // highest such lane (unique unless empty ranges tie; take the top one)
        int b_l = 0, ab_l = above_lane;
        if (lane == src) {
            int j = PER_LANE - 1;
            for (; j > 0; --j) {
                if (ab_l + mine[j] >= keep) break;
                ab_l += mine[j];
            }
            b_l = lane * PER_LANE + j;
        }
        b = __shfl_sync(0xffffffffu, b_l, src);
        ab = __shfl_sync(0xffffffffu, ab_l, src);
    } else {
        // fewer than `keep` entries in all buckets above 0: the threshold is bucket 0
        int total_above = above0 + __shfl_sync(0xffffffffu, suf, 0) - hist[0];
        b = 0;
        ab = total_above;
    }
    bucket = b;
    above = ab;
}

// Fast path, I <= 2048 and I % 8 == 0: the row lives in registers (8 consecutive entries per thread, so
// thread order = index order for the tie rule), histogram searches and prefix sums run on warps.
__global__ __launch_bounds__(kTopkThreads) void act_topk_kernel(uint16_t* __restrict__ yact,
                                                                const int32_t* __restrict__ counts,
                                                                const int32_t* __restrict__ offsets, int e_tot, int I,
                                                                int keep) {
    __shared__ int hist[256];
    __shared__ int sel[4];  // bucket, above, threshold, need_equal
    __shared__ int warp_eq[8];
    const int r = blockIdx.x;
    int lo = 0, hi = e_tot;  // largest e with offsets[e] <= r
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (offsets[mid] <= r) lo = mid; else hi = mid;
    }
    if (r >= offsets[e_tot] || r - offsets[lo] >= counts[lo]) return;
    uint4* row4 = reinterpret_cast<uint4*>(yact + (size_t)r * I);
    const int n_vec = I / 8;
    const bool mine = (int)threadIdx.x < n_vec;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (mine) v = row4[threadIdx.x];
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
    int mag[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        mag[2 * j] = (int)(w[j] & 0x7fffu);
        mag[2 * j + 1] = (int)((w[j] >> 16) & 0x7fffu);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    hist[threadIdx.x] = 0;
    __syncthreads();
    if (mine) {
#pragma unroll
        for (int j = 0; j < 8; ++j) atomicAdd(&hist[mag[j] >> 7], 1);
    }
    __syncthreads();
    if (warp == 0) {
        int b, ab;
        topk_find_bucket<8>(hist, keep, 0, b, ab);
        if (lane == 0) { sel[0] = b; sel[1] = ab; }
    }
    __syncthreads();
    const int bucket = sel[0], above1 = sel[1];
    __syncthreads();
    hist[threadIdx.x] = 0;
    __syncthreads();
    if (mine) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if ((mag[j] >> 7) == bucket) atomicAdd(&hist[mag[j] & 127], 1);
    }
    __syncthreads();
    if (warp == 0) {
        int b, ab;
        topk_find_bucket<4>(hist, keep, above1, b, ab);
        if (lane == 0) { sel[2] = (bucket << 7) | b; sel[3] = keep - ab; }
    }
    __syncthreads();
    const int thr = sel[2], need_equal = sel[3];
    // entries equal to the threshold: the first need_equal in index order survive
    int eq = 0;
    if (mine) {
#pragma unroll
        for (int j = 0; j < 8; ++j) eq += mag[j] == thr;
    }
    int incl = eq;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += o;
    }
    if (lane == 31) warp_eq[warp] = incl;
    __syncthreads();
    int before = incl - eq;
    for (int q = 0; q < warp; ++q) before += warp_eq[q];
    if (!mine) return;
    int quota = need_equal - before;
    bool changed = false;
    uint16_t out[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint16_t raw = (uint16_t)(j & 1 ? w[j >> 1] >> 16 : w[j >> 1] & 0xffffu);
        bool keep_it = mag[j] > thr;
        if (mag[j] == thr && quota > 0) {
            --quota;
            keep_it = true;
        }
        out[j] = keep_it ? raw : (uint16_t)0;
        changed |= !keep_it && raw != 0;
    }
    if (changed) {
        uint4 o;
        o.x = out[0] | ((uint32_t)out[1] << 16);
        o.y = out[2] | ((uint32_t)out[3] << 16);
        o.z = out[4] | ((uint32_t)out[5] << 16);
        o.w = out[6] | ((uint32_t)out[7] << 16);
        row4[threadIdx.x] = o;
    }
}

// Warp-per-row path, I = 256 * VEC (VEC 16-byte pieces per lane, read coalesced): no block-wide barriers, eight rows
// of a CTA progress independently. Histograms live in a per-warp slice of shared memory; the two bucket searches
// are the warp routine above. The row is read once into registers and only pieces that change are written back.
// Ties at the threshold: the common case (every entry equal to the threshold survives) needs no ordering; otherwise
// the entries are ranked in index order, which for the coalesced layout is (piece, lane, position in the piece).
template <int VEC>
__global__ __launch_bounds__(kTopkThreads) void act_topk_warp_kernel(uint16_t* __restrict__ yact,
                                                                     const int32_t* __restrict__ counts,
                                                                     const int32_t* __restrict__ offsets, int e_tot,
                                                                     int keep, int max_rows) {
    __shared__ int hist_all[8][256];
    __shared__ int s_off[kTopkMaxExperts + 1], s_cnt[kTopkMaxExperts];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int* hist = hist_all[warp];
    // expert segments once per CTA in shared memory: which rows are padding is then a search without global loads
    for (int e = threadIdx.x; e <= e_tot; e += blockDim.x) {
        s_off[e] = offsets[e];
        if (e < e_tot) s_cnt[e] = counts[e];
    }
    __syncthreads();
    const int r_end = min(max_rows, s_off[e_tot]);
    constexpr int I = 256 * VEC;
    for (int r = blockIdx.x * 8 + warp; r < r_end; r += gridDim.x * 8) {
    int lo = 0, hi = e_tot;  // largest e with offsets[e] <= r
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_off[mid] <= r) lo = mid; else hi = mid;
    }
    if (r - s_off[lo] >= s_cnt[lo]) continue;  // a padding row
    uint4* row4 = reinterpret_cast<uint4*>(yact + (size_t)r * I);
    uint32_t w[VEC][4];
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
        const uint4 q = row4[v * 32 + lane];
        w[v][0] = q.x; w[v][1] = q.y; w[v][2] = q.z; w[v][3] = q.w;
    }
    // Level 1 = the bf16 exponent (top 8 of the 15 magnitude bits). A row's exponents sit in a handful of values
    // (shared-memory atomics on them serialise), and the threshold is almost always within eight exponents of the
    // row's largest: count those eight per lane in one packed 64-bit register, add them up over the warp.
    uint32_t mmax2 = 0u;  // largest magnitude of either half (packed 16-bit max); its exponent is the row's largest
#pragma unroll
    for (int v = 0; v < VEC; ++v)
#pragma unroll
        for (int j = 0; j < 4; ++j) mmax2 = __vmaxu2(mmax2, w[v][j] & 0x7fff7fffu);
    const uint32_t emax = __reduce_max_sync(0xffffffffu, max(mmax2 & 0xffffu, mmax2 >> 16)) >> 7;
    unsigned long long packed = 0ull;  // byte d = this lane's entries with exponent emax - d (a lane holds 8 * VEC <= 128)
#pragma unroll
    for (int v = 0; v < VEC; ++v)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t d0 = emax - ((w[v][j] >> 7) & 0xffu), d1 = emax - ((w[v][j] >> 23) & 0xffu);
            if (d0 < 8u) packed += 1ull << (8u * d0);
            if (d1 < 8u) packed += 1ull << (8u * d1);
        }
    int bucket = -1, above1 = 0;
#pragma unroll
    for (int d = 0; d < 8; ++d) {
        const int tot = __reduce_add_sync(0xffffffffu, (int)((packed >> (8 * d)) & 0xffull));
        if (bucket < 0) {
            if (above1 + tot >= keep || emax == (uint32_t)d) bucket = (int)emax - d;  // exponent 0 is the last bucket
            else above1 += tot;
        }
    }
    if (bucket < 0) {  // a heavy-tailed row: the general histogram over all 256 exponents
#pragma unroll
        for (int j = 0; j < 8; ++j) hist[lane * 8 + j] = 0;
        __syncwarp();
#pragma unroll
        for (int v = 0; v < VEC; ++v)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                atomicAdd(&hist[(w[v][j] & 0x7fffu) >> 7], 1);
                atomicAdd(&hist[(w[v][j] >> 23) & 0xffu], 1);
            }
        __syncwarp();
        topk_find_bucket<8>(hist, keep, 0, bucket, above1);
        __syncwarp();
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) hist[lane * 4 + j] = 0;
    __syncwarp();
#pragma unroll
    for (int v = 0; v < VEC; ++v)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m0 = (int)(w[v][j] & 0x7fffu), m1 = (int)((w[v][j] >> 16) & 0x7fffu);
            if ((m0 >> 7) == bucket) atomicAdd(&hist[m0 & 127], 1);
            if ((m1 >> 7) == bucket) atomicAdd(&hist[m1 & 127], 1);
        }
    __syncwarp();
    int b2, above2;
    topk_find_bucket<4>(hist, keep, above1, b2, above2);
    const int thr = (bucket << 7) | b2;
    const int need_equal = keep - above2;  // entries equal to the threshold that survive (the first ones in index order)
    // entries equal to the threshold, per piece
    int eq[VEC], eq_lane = 0;
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
        int c = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            c += ((int)(w[v][j] & 0x7fffu) == thr) + ((int)((w[v][j] >> 16) & 0x7fffu) == thr);
        eq[v] = c;
        eq_lane += c;
    }
    const int eq_total = __reduce_add_sync(0xffffffffu, eq_lane);
    const bool all_ties_survive = eq_total <= need_equal;
    int before_piece = 0;  // slow path: threshold entries in earlier pieces (all lanes)
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
        int quota = 1 << 30;
        if (!all_ties_survive) {
            int incl = eq[v];
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int o = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += o;
            }
            quota = need_equal - before_piece - (incl - eq[v]);
            before_piece += __shfl_sync(0xffffffffu, incl, 31);
        }
        uint32_t o[4];
        bool changed = false;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t word = w[v][j];
            const int m0 = (int)(word & 0x7fffu), m1 = (int)((word >> 16) & 0x7fffu);
            bool k0 = m0 > thr, k1 = m1 > thr;
            if (m0 == thr && quota > 0) { --quota; k0 = true; }
            if (m1 == thr && quota > 0) { --quota; k1 = true; }
            if (!k0) word &= 0xffff0000u;
            if (!k1) word &= 0x0000ffffu;
            changed |= word != w[v][j];
            o[j] = word;
        }
        if (changed) row4[v * 32 + lane] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    __syncwarp();
    }  // rows of this warp
}

template <int VEC>
void launch_act_topk_warp(const ActTopkArgs& a, cudaStream_t stream) {
    int blocks = (a.max_rows + 7) / 8;
    if (blocks > 148 * 8) blocks = 148 * 8;  // warps walk the rows with a stride
    act_topk_warp_kernel<VEC><<<blocks, kTopkThreads, 0, stream>>>((uint16_t*)a.yact, a.counts, a.offsets, a.E_tot,
                                                                   a.keep, a.max_rows);
}

int launch_act_topk(const ActTopkArgs& a, cudaStream_t stream) {
    if (a.keep <= 0 || a.keep >= a.I || a.max_rows <= 0) return XMOE_OK;
    if (a.E_tot > kTopkMaxExperts) return XMOE_ERR_SHAPE;
    if (a.I == 512) launch_act_topk_warp<2>(a, stream);
    else if (a.I == 1024) launch_act_topk_warp<4>(a, stream);
    else if (a.I == 2048) launch_act_topk_warp<8>(a, stream);
    else if (a.I == 4096) launch_act_topk_warp<16>(a, stream);
    else if (a.I <= 8 * kTopkThreads && a.I % 8 == 0)
        act_topk_kernel<<<a.max_rows, kTopkThreads, 0, stream>>>((uint16_t*)a.yact, a.counts, a.offsets, a.E_tot, a.I,
                                                                 a.keep);
    else
        act_topk_general_kernel<<<a.max_rows, kTopkThreads, 0, stream>>>((uint16_t*)a.yact, a.counts, a.offsets, a.E_tot,
                                                                         a.I, a.keep);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

// ------------------------------------------------------------------------------------
// Weight preparation (load time).
// ------------------------------------------------------------------------------------
// E4M3 block scales [n_mats, rows, kblocks16] (checkpoint order, one byte per 16 K) ->
// [n_mats, mb, kb_pad, 512]: per 128-row block and 64-K block one 512-byte tile holding
// byte (row%32)*16 + (row/32 % 4)*4 + (k16 % 4); rows/K beyond the matrix are zero.
__global__ void prep_nvfp4_sf_kernel(const uint8_t* __restrict__ in, uint32_t* __restrict__ out, size_t n_words,
                                     int rows, int kblocks16, int mb, int kb_pad) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += (size_t)gridDim.x * blockDim.x) {
        const int word = (int)(i % 128);  // 128 words per 512-byte tile
        size_t tile = i / 128;
        const int kb = (int)(tile % kb_pad);
        tile /= kb_pad;
        const int rb = (int)(tile % mb);
        const size_t mat = tile / mb;
        const int r32 = word >> 2, c4 = word & 3;
        const int row = rb * 128 + c4 * 32 + r32;
        uint32_t v = 0u;
        if (row < rows) {
            const uint8_t* src = in + ((size_t)mat * rows + row) * kblocks16;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int k16 = kb * 4 + j;
                if (k16 < kblocks16) v |= (uint32_t)src[k16] << (8 * j);
            }
        }
        out[i] = v;
    }
}

int launch_prep_nvfp4_sf(const void* sf_in, void* sf_out, int n_mats, int rows, int kblocks16, int mb, int kb_pad,
                         cudaStream_t stream) {
    const size_t n_words = (size_t)n_mats * mb * kb_pad * 128;
    if (!n_words) return XMOE_OK;
    size_t blocks = (n_words + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    prep_nvfp4_sf_kernel<<<(int)blocks, 256, 0, stream>>>((const uint8_t*)sf_in, (uint32_t*)sf_out, n_words, rows,
                                                          kblocks16, mb, kb_pad);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

// Pair-interleaved nibble order used by the FF2 dequantiser: inside each 32-bit word
// (8 consecutive K) nibble j holds K 2j and nibble 4+j holds K 2j+1, so that
// (word >> 4j) & 0x000f000f is the bf16x2 pair (K 2j, K 2j+1) without any permute.
__device__ __forceinline__ uint32_t interleave_pairs(uint32_t lin) {
    uint32_t o = 0u;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        o |= ((lin >> (8 * j)) & 0xfu) << (4 * j);
        o |= ((lin >> (8 * j + 4)) & 0xfu) << (16 + 4 * j);
    }
    return o;
}

// GPTQ int32 [E, K/8, O] (uint4b8, nibble j of word (k8, o) is K index 8*k8 + j; the same
// input contract as the reference repack xR64ABSRepack.cu:3-24) -> K-major words
// [E, O, K/8] in pair-interleaved order, values kept offset-binary (u4 = q + 8).
__global__ void repack_gptq_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, size_t n_words, int K8,
                                   int O) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += (size_t)gridDim.x * blockDim.x) {
        const int o = (int)(i % O);
        size_t rest = i / O;
        const int k8 = (int)(rest % K8);
        const size_t e = rest / K8;
        out[((size_t)e * O + o) * K8 + k8] = interleave_pairs(in[i]);
    }
}

int launch_repack_gptq(const void* qweight, void* out, int E, int K, int O, cudaStream_t stream) {
    if (K % 8) return XMOE_ERR_SHAPE;
    const size_t n_words = (size_t)E * (K / 8) * O;
    if (!n_words) return XMOE_OK;
    size_t blocks = (n_words + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    repack_gptq_kernel<<<(int)blocks, 256, 0, stream>>>((const uint32_t*)qweight, (uint32_t*)out, n_words, K / 8, O);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

// K-major words in linear nibble order (low nibble = lower K) -> pair-interleaved order.
__global__ void repack_kmajor_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, size_t n_words) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += (size_t)gridDim.x * blockDim.x)
        out[i] = interleave_pairs(in[i]);
}

int launch_repack_kmajor_int4(const void* w_in, void* out, size_t n_words, cudaStream_t stream) {
    if (!n_words) return XMOE_OK;
    size_t blocks = (n_words + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    repack_kmajor_kernel<<<(int)blocks, 256, 0, stream>>>((const uint32_t*)w_in, (uint32_t*)out, n_words);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

}  // namespace xmoe
