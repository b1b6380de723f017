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

int launch_act_topk(const ActTopkArgs& a, cudaStream_t stream) {
    if (a.keep <= 0 || a.keep >= a.I || a.max_rows <= 0) return XMOE_OK;
    if (a.I <= 8 * kTopkThreads && a.I % 8 == 0)
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
