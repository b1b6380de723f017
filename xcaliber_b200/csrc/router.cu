// Router (top-k selection + gate weights) and the deterministic expert-contiguous
// permutation ("route pack").
//
// Semantics follow the reference router xFused-NVFP4-Kernels/xMoE/xW4A16/sm120a/topk.cuh:25-142
// (selection on the ordered bf16 bit pattern, ties to the lower expert id, slots in
// descending logit order, weights normalised over the selected k) and the reference
// permutation .../sm120a/preamble.cuh:466-535 (per expert, rows in ascending token
// order). The permutation here costs O(N*k) instead of the reference's O(E*N*k): a
// per-chunk histogram, a scan, and an in-order rank assignment per warp.
#include "common.cuh"
#include "kernels.h"
#include "router_core.cuh"

namespace xmoe {

// ------------------------------------------------------------------------------------
// Flat top-k on bf16 logits (softmax or sigmoid weights). One warp per token, lane l
// owns experts l + 32*j; every composite key lives in a register, so logits are read
// from HBM exactly once.
// ------------------------------------------------------------------------------------
template <bool SIGMOID, int J>
__global__ __launch_bounds__(256) void router_topk_flat_kernel(
    const uint16_t* __restrict__ logits, const uint16_t* __restrict__ expert_scale,
    int32_t* __restrict__ topk_idx, uint16_t* __restrict__ topk_w,
    int N, int E, int topk, int idx_stride, float routed_scale, int renorm) {
    const uint32_t token = blockIdx.x * 8u + (threadIdx.x >> 5);
    if (token >= (uint32_t)N) return;
    route_token_flat<SIGMOID, J>(logits + (size_t)token * E, lane_id(), token, expert_scale, topk_idx, topk_w, E, topk,
                                 idx_stride, routed_scale, renorm);
}

// Group-limited sigmoid routing with a selection bias: route_token_grouped (router_core.cuh)
template <int J>
__global__ __launch_bounds__(256) void router_topk_grouped_kernel(
    const uint16_t* __restrict__ logits, const float* __restrict__ lut, const float* __restrict__ bias,
    const uint16_t* __restrict__ expert_scale, int32_t* __restrict__ topk_idx, uint16_t* __restrict__ topk_w,
    int N, int E, int topk, int idx_stride, int n_group, int topk_group, float routed_scale, int renorm) {
    const uint32_t token = blockIdx.x * 8u + (threadIdx.x >> 5);
    if (token >= (uint32_t)N) return;
    route_token_grouped<J>(logits + (size_t)token * E, lane_id(), token, lut, bias, expert_scale, topk_idx, topk_w, E,
                           topk, idx_stride, n_group, topk_group, routed_scale, renorm);
}

// ------------------------------------------------------------------------------------
// Route pack. Chunk = 256 tokens per CTA (8 warps x 32 tokens).
//   pass A: per-chunk expert histogram -> chunk_hist[chunk][E_tot]
//   pass B: every CTA rebuilds totals, the 128-row-aligned expert offsets and its own
//           chunk base, then each warp walks its 32 tokens in order handing out ranks.
// Shared experts (ids E .. E+n_shared-1) take every token with weight 1.0 in the extra
// slots topk .. topk+n_shared-1.
// ------------------------------------------------------------------------------------
constexpr int kPackChunk = 256;
constexpr int kMaxEtot = 1024 + 8;

// n_valid (optional, device): only the first *n_valid tokens are in use (an expert-parallel receive buffer sized for
// the worst case); chunks beyond them do nothing, and their rows of the index arrays are left as they are.
__global__ __launch_bounds__(256) void route_hist_kernel(const int32_t* __restrict__ topk_idx, int N, int E,
                                                         int topk, int idx_stride, int n_shared,
                                                         int32_t* __restrict__ chunk_hist,
                                                         const int32_t* __restrict__ n_valid) {
    __shared__ int hist[kMaxEtot];
    if (n_valid) N = min(N, max(*n_valid, 0));
    if ((int)blockIdx.x * kPackChunk >= N) return;  // the scatter pass only reads the chunks that hold tokens
    const int e_tot = E + n_shared;
    for (int e = threadIdx.x; e < e_tot; e += blockDim.x) hist[e] = 0;
    __syncthreads();
    const int t = blockIdx.x * kPackChunk + threadIdx.x;
    if (t < N) {
        for (int k = 0; k < topk; ++k) {
            const int e = topk_idx[(size_t)t * idx_stride + k];
            if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
        }
        for (int s = 0; s < n_shared; ++s) atomicAdd(&hist[E + s], 1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < e_tot; e += blockDim.x) chunk_hist[(size_t)blockIdx.x * e_tot + e] = hist[e];
}

__global__ __launch_bounds__(256) void route_scatter_kernel(
    int32_t* __restrict__ topk_idx, uint16_t* __restrict__ topk_w, int N, int E, int topk, int idx_stride,
    int n_shared, const int32_t* __restrict__ chunk_hist, int n_chunks, int32_t* __restrict__ counts,
    int32_t* __restrict__ offsets, int32_t* __restrict__ topk_off, int32_t* __restrict__ topk_row,
    int32_t* __restrict__ row_token, uint16_t* __restrict__ row_weight, uint32_t* __restrict__ status,
    const int32_t* __restrict__ n_valid) {
    if (n_valid) {
        N = min(N, max(*n_valid, 0));
        if (n_chunks > 1) n_chunks = max(1, (N + kPackChunk - 1) / kPackChunk);
        if ((int)blockIdx.x >= n_chunks) return;  // chunk 0 always runs: it writes the counts and offsets
    }
    __shared__ int total[kMaxEtot];
    __shared__ int before_chunk[kMaxEtot];
    __shared__ int start[kMaxEtot + 1];
    __shared__ int warp_base[8][kMaxEtot];
    __shared__ int carry;
    const int e_tot = E + n_shared;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunk = blockIdx.x;

    // per-warp histograms of this chunk (later turned into bases in place)
    for (int e = threadIdx.x; e < e_tot; e += blockDim.x)
        for (int w = 0; w < 8; ++w) warp_base[w][e] = 0;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    const int t_mine = chunk * kPackChunk + threadIdx.x;
    if (t_mine < N) {
        for (int k = 0; k < topk; ++k) {
            const int e = topk_idx[(size_t)t_mine * idx_stride + k];
            if (e >= 0 && e < E) atomicAdd(&warp_base[warp][e], 1);
            else if (e != -1) atomicExch(status, 0x600u);  // expert id outside [0, E); -1 = slot not in use
        }
        for (int s = 0; s < n_shared; ++s) atomicAdd(&warp_base[warp][E + s], 1);
    }
    __syncthreads();

    // totals and this chunk's base (tokens of earlier chunks come first). A single chunk is its own
    // total: small batches skip the histogram kernel altogether.
    for (int e = threadIdx.x; e < e_tot; e += blockDim.x) {
        int tot = 0, before = 0;
        if (n_chunks == 1) {
            for (int w = 0; w < 8; ++w) tot += warp_base[w][e];
        } else {
            for (int c = 0; c < n_chunks; ++c) {
                const int h = chunk_hist[(size_t)c * e_tot + e];
                tot += h;
                if (c < chunk) before += h;
            }
        }
        total[e] = tot;
        before_chunk[e] = before;
    }
    __syncthreads();

    // exclusive scan of round_up(total, 128) -> start[]
    if (warp == 0) {
        for (int base = 0; base < e_tot; base += 32) {
            const int e = base + lane;
            const int v = e < e_tot ? ((total[e] + 127) & ~127) : 0;
            int incl = v;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int o = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += o;
            }
            const int c = carry;
            if (e < e_tot) start[e] = c + incl - v;
            __syncwarp();
            if (lane == 31) carry = c + incl;
            __syncwarp();
        }
        if (lane == 0) start[e_tot] = carry;
    }
    __syncthreads();
    if (chunk == 0) {
        for (int e = threadIdx.x; e < e_tot; e += blockDim.x) {
            counts[e] = total[e];
            offsets[e] = start[e];
        }
        if (threadIdx.x == 0) offsets[e_tot] = start[e_tot];
    }
    for (int e = threadIdx.x; e < e_tot; e += blockDim.x) {
        int run = before_chunk[e];  // rows of earlier chunks
        for (int w = 0; w < 8; ++w) {
            const int h = warp_base[w][e];
            warp_base[w][e] = run;
            run += h;
        }
    }
    __syncthreads();

    // in-order rank assignment: a warp walks its 32 tokens; lane k owns slot k. The walk is serial (a token's rank
    // depends on the tokens before it), so its inputs are fetched up front, 32 independent loads per lane, instead of
    // one dependent global load per step.
    const int k_eff = topk + n_shared;
    const int t_first = chunk * kPackChunk + warp * 32;
    int e_pre[32];
    uint16_t w_pre[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        e_pre[i] = -1;
        w_pre[i] = 0;
        if (lane < topk && t_first + i < N) {
            e_pre[i] = topk_idx[(size_t)(t_first + i) * idx_stride + lane];
            w_pre[i] = topk_w[(size_t)(t_first + i) * idx_stride + lane];
        }
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const int t = t_first + i;
        if (t >= N) break;
        if (lane < k_eff) {
            int e;
            uint16_t w;
            if (lane < topk) {
                e = e_pre[i];
                w = w_pre[i];
            } else {
                e = E + (lane - topk);
                w = 0x3f80u;  // 1.0 in bf16
                topk_idx[(size_t)t * idx_stride + lane] = e;
                topk_w[(size_t)t * idx_stride + lane] = w;
            }
            // a caller slot is valid under the same test as the histograms (ids in [E, e_tot) belong to the
            // shared experts' own slots and were never counted for a caller slot)
            if (e >= 0 && e < (lane < topk ? E : e_tot)) {
                const int p = warp_base[warp][e];
                warp_base[warp][e] = p + 1;
                const int r = start[e] + p;
                topk_off[(size_t)t * idx_stride + lane] = p;
                topk_row[(size_t)t * idx_stride + lane] = r;
                row_token[r] = t;
                row_weight[r] = w;
            } else {
                topk_off[(size_t)t * idx_stride + lane] = -1;
                topk_row[(size_t)t * idx_stride + lane] = -1;
            }
        }
        __syncwarp();
    }
}

// ---- host launchers ---------------------------------------------------------------
int launch_router_topk(const RouterArgs& a, cudaStream_t stream) {
    if (a.N <= 0) return XMOE_OK;
    const int k_eff = a.idx_stride;
    dim3 grid((a.N + 7) / 8), block(256);
    const uint16_t* logits = (const uint16_t*)a.logits;
    const uint16_t* es = (const uint16_t*)a.expert_scale;
    if (a.n_group > 1 || a.bias != nullptr) {
        if (a.scoring != 1 || a.lut == nullptr) return XMOE_ERR_SHAPE;
        if (a.n_group < 1 || a.n_group > 32 || a.E % a.n_group) return XMOE_ERR_SHAPE;
        if (a.n_group > 1 && (a.E / a.n_group < 2 || a.topk_group < 1 || a.topk_group > a.n_group ||
                              a.topk > a.topk_group * (a.E / a.n_group)))
            return XMOE_ERR_SHAPE;
        if (a.E <= 256)
            router_topk_grouped_kernel<8><<<grid, block, 0, stream>>>(logits, a.lut, a.bias, es, a.topk_idx,
                                                               (uint16_t*)a.topk_w, a.N, a.E, a.topk, k_eff,
                                                               a.n_group, a.topk_group, a.routed_scale, a.renorm);
        else
            router_topk_grouped_kernel<32><<<grid, block, 0, stream>>>(logits, a.lut, a.bias, es, a.topk_idx,
                                                               (uint16_t*)a.topk_w, a.N, a.E, a.topk, k_eff,
                                                               a.n_group, a.topk_group, a.routed_scale, a.renorm);
    } else {
        // slots per lane: the smallest of 1, 2, 4, 8, 32 that holds E / 32
#define XMOE_FLAT(SIG, J)                                                                                          \
    router_topk_flat_kernel<SIG, J><<<grid, block, 0, stream>>>(logits, es, a.topk_idx, (uint16_t*)a.topk_w, a.N, a.E, \
                                                                a.topk, k_eff, a.routed_scale, a.renorm)
#define XMOE_FLAT_J(SIG)                  \
    do {                                  \
        if (a.E <= 32) XMOE_FLAT(SIG, 1);      \
        else if (a.E <= 64) XMOE_FLAT(SIG, 2);  \
        else if (a.E <= 128) XMOE_FLAT(SIG, 4); \
        else if (a.E <= 256) XMOE_FLAT(SIG, 8); \
        else XMOE_FLAT(SIG, 32);                \
    } while (0)
        if (a.scoring == 1) XMOE_FLAT_J(true);
        else XMOE_FLAT_J(false);
#undef XMOE_FLAT_J
#undef XMOE_FLAT
    }
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

int route_pack_chunks(int N) { return (N + kPackChunk - 1) / kPackChunk; }

int launch_route_pack(const PackArgs& a, cudaStream_t stream) {
    if (a.N <= 0) return XMOE_OK;
    if (a.E + a.n_shared > kMaxEtot || a.topk + a.n_shared > 32) return XMOE_ERR_SHAPE;
    const int chunks = route_pack_chunks(a.N);
    if (chunks > 1)  // a single chunk builds its totals inside the scatter kernel
        route_hist_kernel<<<chunks, 256, 0, stream>>>(a.topk_idx, a.N, a.E, a.topk, a.idx_stride, a.n_shared,
                                                      a.chunk_hist, a.n_valid);
    route_scatter_kernel<<<chunks, 256, 0, stream>>>(a.topk_idx, (uint16_t*)a.topk_w, a.N, a.E, a.topk,
                                                     a.idx_stride, a.n_shared, a.chunk_hist, chunks, a.counts,
                                                     a.offsets, a.topk_off, a.topk_row, a.row_token,
                                                     (uint16_t*)a.row_weight, a.status, a.n_valid);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

// ------------------------------------------------------------------------------------
// Route pack for callers that must not allocate device memory.
//
// The per-chunk histograms normally live in caller-provided scratch. Some callers cannot
// provide any: a serving engine that has already handed every free byte of the GPU to its
// KV-cache pool, or a runtime that routes between layers where cudaMalloc is off limits
// because it may synchronise the device. For them the scratch is this fixed array, which
// every GPU that loads the library holds until the process exits (264,192 bytes).
// It is sized for at most kStaticPackMaxTokens tokens and kMaxEtot experts; the entry
// point refuses larger problems. Nothing in it has to start at zero (pass A overwrites
// every entry pass B reads), but all calls share it: two calls that overlap on the GPU
// (different streams, or a graph replay racing a direct call) corrupt each other.
// ------------------------------------------------------------------------------------
constexpr int kStaticPackMaxTokens = 16384;
constexpr int kStaticPackChunks = kStaticPackMaxTokens / kPackChunk;  // 64
static __device__ __align__(256) int32_t g_static_pack_scratch[kStaticPackChunks * kMaxEtot];

int route_pack_static_max_tokens() { return kStaticPackMaxTokens; }

int launch_route_pack_static(PackArgs a, cudaStream_t stream) {
    if (a.N > kStaticPackMaxTokens) return XMOE_ERR_LIMIT;
    if (a.E + a.n_shared > kMaxEtot) return XMOE_ERR_LIMIT;
    // In host code the array's name is not a device address. Ask the runtime for the address
    // once per device, with that device current, and hand the kernels the result.
    static int32_t* device_ptr[kMaxDevices] = {};
    const int dev = device_slot();
    if (dev < 0) return XMOE_ERR_CUDA;
    if (device_ptr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_pack_scratch) != cudaSuccess || p == nullptr) return XMOE_ERR_CUDA;
        device_ptr[dev] = static_cast<int32_t*>(p);
    }
    a.chunk_hist = device_ptr[dev];
    return launch_route_pack(a, stream);
}

}  // namespace xmoe
