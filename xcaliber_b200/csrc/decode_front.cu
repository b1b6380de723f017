// The front of the layer for decode-sized batches in ONE launch: activation amax and scale, router top-k, the
// expert-contiguous permutation and the NVFP4 activation packets. With a few tokens each of the three kernels it
// replaces (router.cu: router_topk_*, route_scatter; act_quant.cu: act_quant_pack) is a chain of two or three
// memory latencies behind a launch, and together they took as long as a quarter of the weight streaming.
//
// No CTA waits for another one: every CTA repeats the cheap part (the amax over the few hundred KB of x, the
// routing of all N <= 32 tokens, the serial rank walk) in its own shared memory, then quantises its share of the
// (token, 512 K) units; CTA 0 also writes the routing arrays the later kernels read. Same routines, same order of
// operations as the separate kernels, so the same bits: route_token_* from router_core.cuh, the rank walk in token
// order as route_scatter_kernel does it, nvfp4_quantise16 from nvfp4_quant.cuh.
#include "common.cuh"
#include "kernels.h"
#include "nvfp4_quant.cuh"
#include "router_core.cuh"

namespace xmoe {

namespace {

constexpr int kFrontTokens = 32;   // at most this many tokens
constexpr int kFrontSlots = 16;    // top_k + shared experts
constexpr int kFrontMaxEtot = 1024 + 8;

// SIGMOID: flat sigmoid instead of flat softmax weights (group-limited routing keeps the separate kernels: repeated in
// every CTA it costs more than the launches saved). J: router slots per lane (8 for E <= 256, else 32).
template <bool SIGMOID, int J>
__global__ __launch_bounds__(256) void decode_front_kernel(const FrontArgs a) {
    __shared__ int s_cnt[kFrontMaxEtot];        // rows per expert, then the running rank of the walk
    __shared__ int s_start[kFrontMaxEtot + 1];  // first packed row of every expert (multiples of 128)
    __shared__ int32_t s_idx[kFrontTokens * kFrontSlots];
    __shared__ uint16_t s_w[kFrontTokens * kFrontSlots];
    __shared__ int32_t s_row[kFrontTokens * kFrontSlots];
    __shared__ uint32_t warp_max[8];
    __shared__ int carry;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int N = a.N, E = a.E, topk = a.topk, k_eff = a.topk + a.n_shared, e_tot = a.E + a.n_shared;
    const bool writer = blockIdx.x == 0;

    // ---- amax of x -> XGS (as act_quant_pack_kernel<true>)
    const uint16_t* x = reinterpret_cast<const uint16_t*>(a.x);
    {
        const size_t n_vec = (size_t)N * a.H / 8;  // H is a multiple of 16
        const uint4* xv = reinterpret_cast<const uint4*>(x);
        uint32_t mx2 = 0u;
        for (size_t i = threadIdx.x; i < n_vec; i += blockDim.x) {
            const uint4 v = xv[i];
            mx2 = __vmaxu2(mx2, v.x & 0x7fff7fffu);
            mx2 = __vmaxu2(mx2, v.y & 0x7fff7fffu);
            mx2 = __vmaxu2(mx2, v.z & 0x7fff7fffu);
            mx2 = __vmaxu2(mx2, v.w & 0x7fff7fffu);
        }
        uint32_t mx = max(mx2 & 0xffffu, mx2 >> 16);
        mx = __reduce_max_sync(0xffffffffu, mx);
        if (lane == 0) warp_max[warp] = mx;
    }
    for (int e = threadIdx.x; e < e_tot; e += blockDim.x) s_cnt[e] = 0;
    if (threadIdx.x == 0) carry = 0;

    // ---- router: warp w takes tokens w, w + 8, ...; results in shared memory, row pitch k_eff
    const uint16_t* logits = reinterpret_cast<const uint16_t*>(a.logits);
    const uint16_t* es = reinterpret_cast<const uint16_t*>(a.expert_scale);
    for (int t = warp; t < N; t += 8) {
        const uint16_t* row = logits + (size_t)t * E;
        route_token_flat<SIGMOID, J>(row, (uint32_t)lane, (uint32_t)t, es, s_idx, s_w, E, topk, k_eff, a.routed_scale, a.renorm);
        if (lane >= topk && lane < k_eff) {  // shared experts: every token, weight 1.0
            s_idx[t * k_eff + lane] = E + (lane - topk);
            s_w[t * k_eff + lane] = 0x3f80u;
        }
    }
    __syncthreads();
    uint32_t mx = warp_max[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) mx = max(mx, warp_max[w]);
    const float amax = bf16_bits_to_f32(mx);
    const float xgs = mx ? 2688.0f / amax : 0.f;
    if (writer && threadIdx.x == 0) {  // as act_amax_kernel's last block
        a.scale->xgs = xgs;
        a.scale->xgs_inv = mx ? bf16_bits_to_f32(f32_to_bf16_bits(amax * (1.0f / 2688.0f))) : 0.f;
        reinterpret_cast<float*>(a.scale)[2] = amax;
    }

    // ---- rows per expert, 128-row-aligned expert segments
    for (int i = threadIdx.x; i < N * k_eff; i += blockDim.x) atomicAdd(&s_cnt[s_idx[i]], 1);
    __syncthreads();
    if (warp == 0) {
        for (int base = 0; base < e_tot; base += 32) {
            const int e = base + lane;
            const int v = e < e_tot ? ((s_cnt[e] + 127) & ~127) : 0;
            int incl = v;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int o = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += o;
            }
            const int c = carry;
            if (e < e_tot) s_start[e] = c + incl - v;
            __syncwarp();
            if (lane == 31) carry = c + incl;
            __syncwarp();
        }
        if (lane == 0) s_start[e_tot] = carry;
    }
    __syncthreads();
    if (writer) {
        for (int e = threadIdx.x; e < e_tot; e += blockDim.x) {
            a.counts[e] = s_cnt[e];
            a.offsets[e] = s_start[e];
        }
        if (threadIdx.x == 0) a.offsets[e_tot] = s_start[e_tot];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < e_tot; e += blockDim.x) s_cnt[e] = 0;  // now the running rank
    __syncthreads();

    // ---- ranks in token order (one warp, lane = slot): rows of an expert are in ascending token order
    if (warp == 0) {
        for (int t = 0; t < N; ++t) {
            if (lane < k_eff) {
                const int e = s_idx[t * k_eff + lane];
                const int p = s_cnt[e];
                s_cnt[e] = p + 1;
                const int r = s_start[e] + p;
                s_row[t * k_eff + lane] = r;
                if (writer) {
                    const size_t o = (size_t)t * k_eff + lane;
                    a.topk_idx[o] = e;
                    a.topk_w[o] = s_w[t * k_eff + lane];
                    a.topk_off[o] = p;
                    a.topk_row[o] = r;
                    a.row_token[r] = t;
                    a.row_weight[r] = s_w[t * k_eff + lane];
                }
            }
            __syncwarp();
        }
    }
    __syncthreads();

    // ---- NVFP4 packets of this CTA's (token, 512 K) units (as act_quant_pack_kernel)
    const int H = a.H;
    const int units_per_token = (a.kb_pad * 64 + 511) / 512;
    const int total_units = N * units_per_token;
    const int h_pad = a.kb_pad * 64;
    for (int unit = blockIdx.x * 8 + warp; unit < total_units; unit += gridDim.x * 8) {
        const int t = unit / units_per_token;
        const int h0 = (unit % units_per_token) * 512 + lane * 16;
        uint32_t w[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (h0 < H) {
            const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * H + h0);
            const uint4 p = __ldg(src), q = __ldg(src + 1);
            w[0] = p.x; w[1] = p.y; w[2] = p.z; w[3] = p.w;
            w[4] = q.x; w[5] = q.y; w[6] = q.z; w[7] = q.w;
        }
        uint32_t sbyte, q_lo, q_hi;
        nvfp4_quantise16(w, xgs, sbyte, q_lo, q_hi);
        uint32_t s4 = sbyte << (8 * (lane & 3));
        s4 |= __shfl_xor_sync(0xffffffffu, s4, 1);
        s4 |= __shfl_xor_sync(0xffffffffu, s4, 2);
        const int kb = h0 >> 6;
        for (int k = 0; k < k_eff; ++k) {
            const int r = s_row[t * k_eff + k];
            if (h0 < H) *reinterpret_cast<uint2*>(a.xq + (size_t)r * (H / 2) + h0 / 2) = make_uint2(q_lo, q_hi);
            if ((lane & 3) == 0 && h0 < h_pad) {
                const size_t blk = (size_t)(r / a.nt) * a.kb_pad + kb;
                *reinterpret_cast<uint32_t*>(a.sfx + blk * 512 + (r & 31) * 16 + ((r % a.nt) >> 5) * 4) = s4;
            }
        }
    }
}

}  // namespace

bool decode_front_applies(int N, int E, int topk, int n_shared, int H) {
    return N >= 1 && N <= kFrontTokens && topk + n_shared <= kFrontSlots && E + n_shared <= kFrontMaxEtot && H % 16 == 0 &&
           (size_t)N * H <= ((size_t)1 << 18);
}

int launch_decode_front(const FrontArgs& a, cudaStream_t stream) {
    if (!decode_front_applies(a.N, a.E, a.topk, a.n_shared, a.H)) return XMOE_ERR_SHAPE;
    if (a.nt != 32 && a.nt != 64 && a.nt != 128) return XMOE_ERR_SHAPE;
    const int units = a.N * ((a.kb_pad * 64 + 511) / 512);
    const int blocks = (units + 7) / 8;
    if (a.E <= 256) {
        if (a.scoring == 1) decode_front_kernel<true, 8><<<blocks, 256, 0, stream>>>(a);
        else decode_front_kernel<false, 8><<<blocks, 256, 0, stream>>>(a);
    } else {
        if (a.scoring == 1) decode_front_kernel<true, 32><<<blocks, 256, 0, stream>>>(a);
        else decode_front_kernel<false, 32><<<blocks, 256, 0, stream>>>(a);
    }
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

}  // namespace xmoe
