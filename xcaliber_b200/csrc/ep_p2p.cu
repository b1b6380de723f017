// Expert-parallel token exchange over peer memory (NVLink / NVSwitch), device side.
//
// Not in the reference (its plugin refuses EP != 1, vllm/xcaliber_int4_vllm/method.py:130-138).
// One process per GPU; every rank maps every other rank's exchange buffers (plain peer
// pointers, no multicast). A layer call is a fixed sequence of kernels on each rank's stream,
// with no host synchronisation and no host-known row counts:
//
//   post_counts   per-destination row counts + local activation amax -> every rank's table
//   dispatch      wait for all tables; copy each (token, slot) row and its (local expert, gate
//                 weight, home slot) record straight into the owner rank's receive buffer, at a
//                 position fixed by (source rank, expert, order inside the expert)
//   wait_data     wait until every rank's rows have landed; expand the records into the
//                 routing arrays of the local pipeline (expert id -1 = unused row)
//   (local route pack -> NVFP4 quantise -> FF1 -> FF2 on the received rows)
//   return        copy each FF2 output row back to its home rank, slot (token * k + slot)
//   wait_ret      wait until every rank has returned its rows; the home rank then sums them
//
// Synchronisation is by epoch-valued flags in each rank's control block: a writer stores data,
// fences at system scope and then releases the flag in the READER's memory; a reader spins on
// its own memory. Every spin is bounded: when it gives up it records XMOE_EP_TIMEOUT in the
// control block and the kernel carries on (on incomplete data) so that the stream drains.
// The flags of one call also fence buffer reuse: nobody starts call t+1 before it has seen
// every rank's return flag of call t, and a rank raises that flag only after its last read of
// its receive buffer and count table.
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "nvfp4_quant.cuh"

namespace xmoe {

namespace {

constexpr int kMaxWorld = 8;
constexpr int kMaxEpExperts = 1024;
constexpr uint32_t kSpinLimit = 1u << 24;  // polls of ~200 ns each: a few seconds (XMOE_EP_SPIN_LIMIT overrides)

struct EpCtl {  // 512 bytes, zero-initialised by the host before the first call
    int32_t counts[kMaxWorld][kMaxWorld];  // [source rank][destination rank] rows
    uint32_t amax[kMaxWorld];              // fp32 bits (non-negative: ordered as integers)
    uint32_t flag_counts[kMaxWorld];
    uint32_t flag_data[kMaxWorld];
    uint32_t flag_ret[kMaxWorld];
    uint32_t epoch;            // local: number of calls started
    uint32_t ticket_dispatch;  // local: CTAs of the dispatch kernel that finished storing
    uint32_t ticket_return;
    uint32_t error;            // local: sticky XMOE_EP_* bits
    uint32_t pad[28];
};
static_assert(sizeof(EpCtl) == XMOE_EP_CTL_BYTES, "control block layout");
static_assert(offsetof(EpCtl, error) == (64 + 8 + 24 + 3) * 4, "xmoe_ep_status reads the error word at this offset");
static_assert(kMaxWorld == XMOE_EP_MAX_WORLD, "public limit");

constexpr uint32_t kErrTimeout = XMOE_EP_TIMEOUT, kErrCapacity = XMOE_EP_CAPACITY, kErrExpert = XMOE_EP_EXPERT;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Bounded wait until *flag has reached `epoch` (wrap-safe).
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch, uint32_t* error, uint32_t limit) {
    for (uint32_t i = 0; i < limit; ++i) {
        if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
        __nanosleep(200);
    }
    atomicOr(error, kErrTimeout);
    return false;
}

struct EpCtx {
    EpCtl* ctl[kMaxWorld];
    uint4* recv_x[kMaxWorld];     // bf16 [cap_rows, H]
    int4* recv_meta[kMaxWorld];   // [cap_rows]: local expert, gate weight bits, home slot, 0
    uint4* ret_rows[kMaxWorld];   // bf16 [ret_cap, H]
    int world, rank, H, experts_per_rank, cap_rows, ret_cap;
    uint32_t spin_limit;  // polls a flag wait makes before it records XMOE_EP_TIMEOUT and carries on
};

__global__ __launch_bounds__(256) void ep_post_counts_kernel(EpCtx c, const int32_t* __restrict__ counts_global,
                                                            const float* __restrict__ amax_local) {
    __shared__ int dest_sum[kMaxWorld];
    __shared__ uint32_t epoch;
    EpCtl* me = c.ctl[c.rank];
    if (threadIdx.x == 0) {
        epoch = me->epoch + 1u;
        me->epoch = epoch;
    }
    if (threadIdx.x < c.world) {
        int s = 0;
        for (int e = 0; e < c.experts_per_rank; ++e) s += counts_global[threadIdx.x * c.experts_per_rank + e];
        dest_sum[threadIdx.x] = s;
    }
    __syncthreads();
    if (threadIdx.x < c.world) {
        EpCtl* peer = c.ctl[threadIdx.x];
        for (int d = 0; d < c.world; ++d) peer->counts[c.rank][d] = dest_sum[d];
        peer->amax[c.rank] = __float_as_uint(amax_local ? fabsf(amax_local[0]) : 0.f);
        __threadfence_system();
        st_release_sys(&peer->flag_counts[c.rank], epoch);
    }
}

// Warp copy of one bf16 row (H % 8 == 0), 16 bytes per lane and step.
__device__ __forceinline__ void copy_row(uint4* dst, const uint4* src, int hv, int lane) {
    for (int i = lane; i < hv; i += 32) dst[i] = src[i];
}

__global__ __launch_bounds__(256) void ep_dispatch_kernel(EpCtx c, const uint4* __restrict__ x,
                                                         const int32_t* __restrict__ topk_idx,
                                                         const uint16_t* __restrict__ topk_w,
                                                         const int32_t* __restrict__ topk_off,
                                                         const int32_t* __restrict__ counts_global, int n, int top_k,
                                                         int idx_stride, float* __restrict__ amax_global) {
    __shared__ int base[kMaxWorld];         // rows of lower ranks ahead of mine at each destination
    __shared__ int pre[kMaxEpExperts];      // rows of earlier experts of the same owner rank (mine only)
    EpCtl* me = c.ctl[c.rank];
    const uint32_t epoch = me->epoch;
    if (threadIdx.x < c.world) wait_flag(&me->flag_counts[threadIdx.x], epoch, &me->error, c.spin_limit);
    __syncthreads();
    const int E = c.world * c.experts_per_rank;
    if (threadIdx.x < c.world) {
        int s = 0;
        for (int r = 0; r < c.rank; ++r) s += me->counts[r][threadIdx.x];
        base[threadIdx.x] = s;
    }
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int first = (e / c.experts_per_rank) * c.experts_per_rank;
        int s = 0;
        for (int q = first; q < e; ++q) s += counts_global[q];
        pre[e] = s;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0 && amax_global) {
        uint32_t m = 0;
        for (int r = 0; r < c.world; ++r) m = max(m, me->amax[r]);
        amax_global[0] = __uint_as_float(m);
    }
    __syncthreads();
    const int hv = c.H / 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total = n * top_k;
    for (int a = blockIdx.x * 8 + warp; a < total; a += gridDim.x * 8) {
        const int t = a / top_k, k = a - t * top_k;
        const int e = topk_idx[(size_t)t * idx_stride + k];
        if (e < 0 || e >= E) {
            if (lane == 0) atomicOr(&me->error, kErrExpert);
            continue;
        }
        const int d = e / c.experts_per_rank;
        const int row = base[d] + pre[e] + topk_off[(size_t)t * idx_stride + k];
        if (row < 0 || row >= c.cap_rows) {
            if (lane == 0) atomicOr(&me->error, kErrCapacity);
            continue;
        }
        copy_row(c.recv_x[d] + (size_t)row * hv, x + (size_t)t * hv, hv, lane);
        if (lane == 0)
            c.recv_meta[d][row] = make_int4(e - d * c.experts_per_rank, (int)topk_w[(size_t)t * idx_stride + k], a, 0);
    }
    // every store of this CTA is ordered before its ticket; the last CTA raises the flags
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t ticket = atomicAdd(&me->ticket_dispatch, 1u);
        if (ticket == gridDim.x - 1) {
            me->ticket_dispatch = 0u;
            __threadfence_system();
            for (int p = 0; p < c.world; ++p) st_release_sys(&c.ctl[p]->flag_data[c.rank], epoch);
        }
    }
}

// Dispatch fused with the activation quantiser: every token is quantised ONCE on its home GPU with
// the scale all ranks agree on (2688 / max over ranks of amax) and its NVFP4 packets (H/2 bytes of
// codes + H/16 block-scale bytes, 3.6x fewer bytes than the bf16 row) are stored straight into the
// owner ranks' receive buffers: codes at [row, H/2], scales at cap_rows * H/2 + [row, H/16] of the same
// region. One warp per (token, 512 K): the arithmetic and its order are act_quant_pack_kernel's.
__global__ __launch_bounds__(256) void ep_dispatch_q_kernel(EpCtx c, const uint16_t* __restrict__ x,
                                                           const int32_t* __restrict__ topk_idx,
                                                           const uint16_t* __restrict__ topk_w,
                                                           const int32_t* __restrict__ topk_off,
                                                           const int32_t* __restrict__ counts_global, int n, int top_k,
                                                           int idx_stride, float* __restrict__ amax_global) {
    __shared__ int base[kMaxWorld];
    __shared__ int pre[kMaxEpExperts];
    __shared__ float xgs_s;
    EpCtl* me = c.ctl[c.rank];
    const uint32_t epoch = me->epoch;
    if (threadIdx.x < c.world) wait_flag(&me->flag_counts[threadIdx.x], epoch, &me->error, c.spin_limit);
    __syncthreads();
    const int E = c.world * c.experts_per_rank;
    if (threadIdx.x < c.world) {
        int s = 0;
        for (int r = 0; r < c.rank; ++r) s += me->counts[r][threadIdx.x];
        base[threadIdx.x] = s;
    }
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int first = (e / c.experts_per_rank) * c.experts_per_rank;
        int s = 0;
        for (int q = first; q < e; ++q) s += counts_global[q];
        pre[e] = s;
    }
    if (threadIdx.x == 0) {
        uint32_t m = 0;
        for (int r = 0; r < c.world; ++r) m = max(m, me->amax[r]);
        const float amax = __uint_as_float(m);
        xgs_s = amax > 0.f ? 2688.0f / amax : 0.f;  // as act_scale_from_amax_kernel
        if (blockIdx.x == 0 && amax_global) amax_global[0] = amax;
    }
    __syncthreads();
    const float xgs = xgs_s;
    const int H = c.H;
    const int units_per_token = (H + 511) / 512;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t sf_base = (size_t)c.cap_rows * (H / 2);
    const size_t total_units = (size_t)n * units_per_token;
    for (size_t unit = (size_t)blockIdx.x * 8 + warp; unit < total_units; unit += (size_t)gridDim.x * 8) {
        const int t = (int)(unit / units_per_token);
        const int u = (int)(unit % units_per_token);
        const int h0 = u * 512 + lane * 16;
        uint32_t w[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (h0 < H) {
            const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * H + h0);
            const uint4 a = src[0], b = src[1];
            w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
            w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
        }
        uint32_t sbyte, q_lo, q_hi;
        nvfp4_quantise16(w, xgs, sbyte, q_lo, q_hi);
        uint32_t s4 = sbyte << (8 * (lane & 3));
        s4 |= __shfl_xor_sync(0xffffffffu, s4, 1);
        s4 |= __shfl_xor_sync(0xffffffffu, s4, 2);
        for (int k = 0; k < top_k; ++k) {
            const int e = topk_idx[(size_t)t * idx_stride + k];
            if (e < 0 || e >= E) {
                if (lane == 0 && u == 0) atomicOr(&me->error, kErrExpert);
                continue;
            }
            const int d = e / c.experts_per_rank;
            const int row = base[d] + pre[e] + topk_off[(size_t)t * idx_stride + k];
            if (row < 0 || row >= c.cap_rows) {
                if (lane == 0 && u == 0) atomicOr(&me->error, kErrCapacity);
                continue;
            }
            uint8_t* dst = reinterpret_cast<uint8_t*>(c.recv_x[d]);
            if (h0 < H) {
                *reinterpret_cast<uint2*>(dst + (size_t)row * (H / 2) + h0 / 2) = make_uint2(q_lo, q_hi);
                if ((lane & 3) == 0) *reinterpret_cast<uint32_t*>(dst + sf_base + (size_t)row * (H / 16) + (h0 >> 4)) = s4;
            }
            if (u == 0 && lane == 0)
                c.recv_meta[d][row] =
                    make_int4(e - d * c.experts_per_rank, (int)topk_w[(size_t)t * idx_stride + k], t * top_k + k, 0);
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t ticket = atomicAdd(&me->ticket_dispatch, 1u);
        if (ticket == gridDim.x - 1) {
            me->ticket_dispatch = 0u;
            __threadfence_system();
            for (int p = 0; p < c.world; ++p) st_release_sys(&c.ctl[p]->flag_data[c.rank], epoch);
        }
    }
}

__global__ __launch_bounds__(256) void ep_wait_data_kernel(EpCtx c, int32_t* __restrict__ e_recv,
                                                          uint16_t* __restrict__ w_recv, int32_t* __restrict__ n_recv) {
    __shared__ int total;
    EpCtl* me = c.ctl[c.rank];
    const uint32_t epoch = me->epoch;
    if (threadIdx.x < c.world) wait_flag(&me->flag_data[threadIdx.x], epoch, &me->error, c.spin_limit);
    __syncthreads();
    if (threadIdx.x == 0) {
        int s = 0;
        for (int r = 0; r < c.world; ++r) s += me->counts[r][c.rank];
        total = min(s, c.cap_rows);
        if (blockIdx.x == 0 && n_recv) n_recv[0] = total;
    }
    __syncthreads();
    const int4* meta = c.recv_meta[c.rank];
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < c.cap_rows; j += gridDim.x * blockDim.x) {
        if (j < total) {
            const int4 m = meta[j];
            e_recv[j] = m.x;
            w_recv[j] = (uint16_t)m.y;
        } else {
            e_recv[j] = -1;
            w_recv[j] = 0;
        }
    }
}

__global__ __launch_bounds__(256) void ep_return_kernel(EpCtx c, const uint4* __restrict__ out_rows,
                                                       const int32_t* __restrict__ topk_row) {
    __shared__ int bound[kMaxWorld + 1];  // receive-buffer regions by source rank
    EpCtl* me = c.ctl[c.rank];
    const uint32_t epoch = me->epoch;
    if (threadIdx.x == 0) {
        int s = 0;
        for (int r = 0; r < c.world; ++r) {
            bound[r] = s;
            s += me->counts[r][c.rank];
        }
        bound[c.world] = min(s, c.cap_rows);
    }
    __syncthreads();
    const int hv = c.H / 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total = bound[c.world];
    const int4* meta = c.recv_meta[c.rank];
    for (int j = blockIdx.x * 8 + warp; j < total; j += gridDim.x * 8) {
        int r = 0;
        while (r + 1 < c.world && j >= bound[r + 1]) ++r;
        const int slot = meta[j].z;
        const int prow = topk_row[j];
        if (slot < 0 || slot >= c.ret_cap || prow < 0) {
            if (lane == 0) atomicOr(&me->error, kErrCapacity);
            continue;
        }
        copy_row(c.ret_rows[r] + (size_t)slot * hv, out_rows + (size_t)prow * hv, hv, lane);
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t ticket = atomicAdd(&me->ticket_return, 1u);
        if (ticket == gridDim.x - 1) {
            me->ticket_return = 0u;
            __threadfence_system();
            for (int p = 0; p < c.world; ++p) st_release_sys(&c.ctl[p]->flag_ret[c.rank], epoch);
        }
    }
}

// Destination of every packed row of the local pipeline: the slot of its home rank's return buffer.
// With this table the FF2 epilogue stores its rows straight into peer memory (no separate return copy).
__global__ __launch_bounds__(256) void ep_row_dst_kernel(EpCtx c, const int32_t* __restrict__ topk_row,
                                                        unsigned long long* __restrict__ row_dst) {
    __shared__ int bound[kMaxWorld + 1];
    EpCtl* me = c.ctl[c.rank];
    if (threadIdx.x == 0) {
        int s = 0;
        for (int r = 0; r < c.world; ++r) {
            bound[r] = s;
            s += me->counts[r][c.rank];
        }
        bound[c.world] = min(s, c.cap_rows);
    }
    __syncthreads();
    const int total = bound[c.world];
    const int4* meta = c.recv_meta[c.rank];
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < total; j += gridDim.x * blockDim.x) {
        int r = 0;
        while (r + 1 < c.world && j >= bound[r + 1]) ++r;
        const int slot = meta[j].z;
        const int prow = topk_row[j];
        if (slot < 0 || slot >= c.ret_cap || prow < 0) {
            atomicOr(&me->error, kErrCapacity);
            continue;
        }
        row_dst[prow] = (unsigned long long)(uintptr_t)c.ret_rows[r] + (unsigned long long)slot * c.H * 2ull;
    }
}

// Raised after the kernel whose stores were the return transfer: stream order puts those stores
// before this kernel, the system fence and the releases publish them to the peers.
__global__ void ep_signal_ret_kernel(EpCtx c) {
    EpCtl* me = c.ctl[c.rank];
    if (threadIdx.x < c.world) {
        __threadfence_system();
        st_release_sys(&c.ctl[threadIdx.x]->flag_ret[c.rank], me->epoch);
    }
}

__global__ void ep_wait_ret_kernel(EpCtx c) {
    EpCtl* me = c.ctl[c.rank];
    if (threadIdx.x < c.world) wait_flag(&me->flag_ret[threadIdx.x], me->epoch, &me->error, c.spin_limit);
}

int make_ctx(const xmoe_ep_buffers* b, EpCtx* c) {
    if (!b || b->world < 1 || b->world > kMaxWorld || b->rank < 0 || b->rank >= b->world) return XMOE_ERR_ARG;
    if (b->hidden <= 0 || b->hidden % 8 || b->experts_per_rank <= 0) return XMOE_ERR_SHAPE;
    if (b->world * b->experts_per_rank > kMaxEpExperts) return XMOE_ERR_LIMIT;
    if (b->cap_rows <= 0 || b->ret_cap <= 0) return XMOE_ERR_ARG;
    for (int r = 0; r < b->world; ++r) {
        if (!b->ctl[r] || !b->recv_x[r] || !b->recv_meta[r] || !b->ret_rows[r]) return XMOE_ERR_ARG;
        c->ctl[r] = (EpCtl*)b->ctl[r];
        c->recv_x[r] = (uint4*)b->recv_x[r];
        c->recv_meta[r] = (int4*)b->recv_meta[r];
        c->ret_rows[r] = (uint4*)b->ret_rows[r];
    }
    c->world = b->world;
    c->rank = b->rank;
    c->H = b->hidden;
    c->experts_per_rank = b->experts_per_rank;
    c->cap_rows = b->cap_rows;
    c->ret_cap = b->ret_cap;
    // XMOE_EP_SPIN_LIMIT (polls, read at every call): lets an operator shorten the few-second default, and
    // lets a test make a wait on a flag that nobody posts run out within a millisecond
    c->spin_limit = kSpinLimit;
    if (const char* env = getenv("XMOE_EP_SPIN_LIMIT")) {
        const long v = atol(env);
        if (v > 0 && v <= (long)kSpinLimit) c->spin_limit = (uint32_t)v;
    }
    return XMOE_OK;
}

int grid_for(int warps_of_work) {
    int blocks = (warps_of_work + 7) / 8;
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 4) blocks = 148 * 4;
    return blocks;
}

}  // namespace

int launch_ep_post_counts(const xmoe_ep_buffers* b, const int32_t* counts_global, const float* amax_local,
                          cudaStream_t stream) {
    EpCtx c;
    int rc = make_ctx(b, &c);
    if (rc) return rc;
    if (!counts_global) return XMOE_ERR_ARG;
    ep_post_counts_kernel<<<1, 256, 0, stream>>>(c, counts_global, amax_local);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

int launch_ep_dispatch(const xmoe_ep_buffers* b, const void* x, const int32_t* topk_idx, const void* topk_w,
                       const int32_t* topk_off, const int32_t* counts_global, int n, int top_k, int idx_stride,
                       float* amax_global, cudaStream_t stream) {
    EpCtx c;
    int rc = make_ctx(b, &c);
    if (rc) return rc;
    if (n < 0 || top_k < 1 || idx_stride < top_k) return XMOE_ERR_ARG;
    if (n > 0 && (!x || !topk_idx || !topk_w || !topk_off)) return XMOE_ERR_ARG;
    if (!counts_global) return XMOE_ERR_ARG;
    if ((long long)n * top_k > b->ret_cap) return XMOE_ERR_LIMIT;
    ep_dispatch_kernel<<<grid_for(n * top_k), 256, 0, stream>>>(c, (const uint4*)x, topk_idx, (const uint16_t*)topk_w,
                                                               topk_off, counts_global, n, top_k, idx_stride,
                                                               amax_global);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

int launch_ep_dispatch_q(const xmoe_ep_buffers* b, const void* x, const int32_t* topk_idx, const void* topk_w,
                         const int32_t* topk_off, const int32_t* counts_global, int n, int top_k, int idx_stride,
                         float* amax_global, cudaStream_t stream) {
    EpCtx c;
    int rc = make_ctx(b, &c);
    if (rc) return rc;
    if (n < 0 || top_k < 1 || idx_stride < top_k) return XMOE_ERR_ARG;
    if (n > 0 && (!x || !topk_idx || !topk_w || !topk_off)) return XMOE_ERR_ARG;
    if (!counts_global) return XMOE_ERR_ARG;
    if (c.H % 64) return XMOE_ERR_SHAPE;
    if ((long long)n * top_k > b->ret_cap) return XMOE_ERR_LIMIT;
    const int units = (c.H + 511) / 512;
    ep_dispatch_q_kernel<<<grid_for(n * units), 256, 0, stream>>>(c, (const uint16_t*)x, topk_idx,
                                                                 (const uint16_t*)topk_w, topk_off, counts_global, n,
                                                                 top_k, idx_stride, amax_global);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

int launch_ep_wait_data(const xmoe_ep_buffers* b, int32_t* e_recv, void* w_recv, int32_t* n_recv,
                        cudaStream_t stream) {
    EpCtx c;
    int rc = make_ctx(b, &c);
    if (rc) return rc;
    if (!e_recv || !w_recv) return XMOE_ERR_ARG;
    int blocks = (c.cap_rows + 255) / 256;
    blocks = blocks > 148 ? 148 : blocks;
    ep_wait_data_kernel<<<blocks, 256, 0, stream>>>(c, e_recv, (uint16_t*)w_recv, n_recv);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

int launch_ep_return(const xmoe_ep_buffers* b, const void* out_rows, const int32_t* topk_row, int expected_rows,
                     cudaStream_t stream) {
    EpCtx c;
    int rc = make_ctx(b, &c);
    if (rc) return rc;
    if (!out_rows || !topk_row) return XMOE_ERR_ARG;
    ep_return_kernel<<<grid_for(expected_rows > 0 ? expected_rows : 1), 256, 0, stream>>>(c, (const uint4*)out_rows,
                                                                                          topk_row);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

int launch_ep_row_dst(const xmoe_ep_buffers* b, const int32_t* topk_row, unsigned long long* row_dst,
                      cudaStream_t stream) {
    EpCtx c;
    int rc = make_ctx(b, &c);
    if (rc) return rc;
    if (!topk_row || !row_dst) return XMOE_ERR_ARG;
    int blocks = (c.cap_rows + 255) / 256;
    blocks = blocks > 148 ? 148 : blocks;
    ep_row_dst_kernel<<<blocks, 256, 0, stream>>>(c, topk_row, row_dst);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

int launch_ep_signal_ret(const xmoe_ep_buffers* b, cudaStream_t stream) {
    EpCtx c;
    int rc = make_ctx(b, &c);
    if (rc) return rc;
    ep_signal_ret_kernel<<<1, 32, 0, stream>>>(c);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

int launch_ep_wait_ret(const xmoe_ep_buffers* b, cudaStream_t stream) {
    EpCtx c;
    int rc = make_ctx(b, &c);
    if (rc) return rc;
    ep_wait_ret_kernel<<<1, 32, 0, stream>>>(c);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

}  // namespace xmoe
