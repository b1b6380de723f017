// FF1 for prefill-sized batches: token-major variant of the NVFP4 W4A4 gate/up GEMM.
//
// Same math and tensor contracts as ff1_nvfp4.cu (reference: xR64FF1FF2/xR64FF1.cu:65-651,
// co-design.md:75-90), different operand roles: 128 packed token rows are the MMA M operand
// and the N operand is 256 wide = 128 gate rows followed by the 128 up rows of the same
// I-range. One tcgen05.mma (M128 N256 K64) per 64 K then produces, for every token lane, the
// gate values in accumulator columns [0,128) and the up values in [128,256): SwiGLU needs no
// exchange between threads, the routing weight is one register per thread, and a thread
// writes 64 contiguous bytes of its own output row per 32 columns (16-byte stores).
//
// Roles: warp 0 TMA producer, warp 1 TMEM owner + MMA issuer, warps 2-9 epilogue.
#include "common.cuh"
#include "kernels.h"
#include "tile_sched.cuh"

namespace xmoe {

#ifdef XMOE_TRACE
// Debug build only: per-CTA, per-tile clock stamps {mma start, mma issued, acc full, epilogue done}.
__device__ unsigned long long g_ff1_trace[148 * 64 * 4];
#define XMOE_TRACE_STAMP(tile, k)                                                              \
    do {                                                                                       \
        if ((tile) < 64u && blockIdx.x < 148u) g_ff1_trace[(blockIdx.x * 64u + (tile)) * 4u + (k)] = clock64(); \
    } while (0)
#else
#define XMOE_TRACE_STAMP(tile, k) do {} while (0)
#endif

namespace {

constexpr int kTokTile = 128;
constexpr int kWTile = 128;            // I rows per tile (per projection)
constexpr int kStageKBytes = 128;      // 256 K elements per stage
constexpr int kKPerStage = 256;
constexpr int kSfBytes = 2048;         // 4 K-blocks x 512-byte scale tile
constexpr int kABytes = kTokTile * kStageKBytes;      // 16 KiB activations
constexpr int kBBytes = 2 * kWTile * kStageKBytes;    // 32 KiB gate|up weights
constexpr int kStageBytes = kABytes + kBBytes + 3 * kSfBytes;   // 54 KiB
constexpr int kStages = 4;
constexpr int kThreads = 416;        // producer warp, MMA warp, 8 epilogue warps, 3 scale-factor copy warps
constexpr int kFirstSfWarp = 10;
constexpr int kTmemCols = 512;
constexpr int kAccCols = 256;
constexpr int kSfSlotCols = 48;        // per stage: 4 K-blocks x (tokens 4 + gate 4 + up 4)
static_assert(kAccCols + kStages * kSfSlotCols <= kTmemCols, "TMEM budget");
constexpr size_t kSmemBytes = 1024 + (size_t)kStages * kStageBytes + 8192;

template <int ACT>
__global__ __launch_bounds__(kThreads, 1) void ff1_nvfp4_prefill_kernel(const __grid_constant__ Ff1Args a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* tail = smem + (size_t)kStages * kStageBytes;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);
    uint64_t* empty_bar = full_bar + 8;
    uint64_t* acc_full = empty_bar + 8;
    uint64_t* acc_empty = acc_full + 1;
    uint64_t* sf_ready = acc_empty + 1;  // [kStages] the three scale-factor copies of the stage are in tensor memory
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sf_ready + 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    int* prefix = reinterpret_cast<int*>(tail + 256);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int w_tiles = a.mb;
    const int k_stages = (a.H + kKPerStage - 1) / kKPerStage;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
            mbar_init(&sf_ready[s], 3);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 8);
        *abort_flag = 0u;
        mbar_fence_init();
        prefetch_tmap(&a.tm_w);
        prefetch_tmap(&a.tm_x);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    if (warp == 2) tile_prefix_build(prefix, a.counts, a.E_tot, w_tiles, kTokTile);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int total_tiles = prefix[a.E_tot];

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < total_tiles && ok; item += gridDim.x) {
                const TileInfo t = tile_decode(item, prefix, a.counts, a.offsets, a.E_tot, kTokTile);
                const int gate_row = t.e * 2 * a.I + t.wt * kWTile;
                const int up_row = gate_row + a.I;
                const uint8_t* sfw_g = a.sfw + ((size_t)(t.e * 2 + 0) * a.mb + t.wt) * a.kb_pad * 512;
                const uint8_t* sfw_u = a.sfw + ((size_t)(t.e * 2 + 1) * a.mb + t.wt) * a.kb_pad * 512;
                const uint8_t* sfx = a.sfx + (size_t)(t.row0 / kTokTile) * a.kb_pad * 512;
                for (int ks = 0; ks < k_stages; ++ks, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1u;
                    if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_MMA)) {
                        ok = false;
                        break;
                    }
                    uint8_t* st = smem + (size_t)s * kStageBytes;
                    mbar_expect_tx(&full_bar[s], kStageBytes);
                    tma_load_2d(st, &a.tm_x, ks * kStageKBytes, t.row0, &full_bar[s]);
                    tma_load_2d(st + kABytes, &a.tm_w, ks * kStageKBytes, gate_row, &full_bar[s]);
                    tma_load_2d(st + kABytes + kWTile * kStageKBytes, &a.tm_w, ks * kStageKBytes, up_row, &full_bar[s]);
                    uint8_t* sf = st + kABytes + kBBytes;
                    tma_load_1d(sf, sfx + (size_t)ks * kSfBytes, kSfBytes, &full_bar[s]);
                    tma_load_1d(sf + kSfBytes, sfw_g + (size_t)ks * kSfBytes, kSfBytes, &full_bar[s]);
                    tma_load_1d(sf + 2 * kSfBytes, sfw_u + (size_t)ks * kSfBytes, kSfBytes, &full_bar[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_nvfp4(kTokTile, 2 * kWTile);
            constexpr uint32_t kStage16 = kStageBytes >> 4;
            const uint32_t a_lo0 = umma_desc_lo_sw128(smem_u32(smem));
            const uint32_t b_lo0 = umma_desc_lo_sw128(smem_u32(smem + kABytes));
            uint32_t tile_n = 0, s = 0, ph = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < total_tiles && ok; item += gridDim.x, ++tile_n) {
                if (!mbar_wait(acc_empty, (tile_n & 1u) ^ 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_EPI)) break;
                tc_fence_after();
                XMOE_TRACE_STAMP(tile_n, 0);
                for (int ks = 0; ks < k_stages; ++ks) {
                    // operands landed (full_bar) and their scale factors are in tensor memory (sf_ready)
                    if (!mbar_wait(&full_bar[s], ph, abort_flag, a.status, XMOE_DEV_TIMEOUT_TMA) ||
                        !mbar_wait(&sf_ready[s], ph, abort_flag, a.status, XMOE_DEV_TIMEOUT_TMA)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sf_tmem = tmem_base + kAccCols + s * kSfSlotCols;
                    const uint32_t a_lo = a_lo0 + s * kStage16;
                    const uint32_t b_lo = b_lo0 + s * kStage16;
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) {
                        mma_nvfp4_lo(tmem_base, a_lo + kb * 2, b_lo + kb * 2, idesc, sf_tmem + kb * 4,
                                     sf_tmem + 16 + kb * 8, (ks | kb) ? 1u : 0u);
                    }
                    tc_commit(&empty_bar[s]);
                    if (++s == (uint32_t)kStages) { s = 0; ph ^= 1u; }
                }
                if (ok) tc_commit(acc_full);
                XMOE_TRACE_STAMP(tile_n, 1);
            }
        }
    } else if (warp >= kFirstSfWarp) {
        // Scale-factor copies, shared memory -> tensor memory, one thread per operand (tokens, gate
        // rows, up rows). A thread issues at most one tcgen05 instruction per ~65 cycles; with the
        // 12 copies of a stage on the MMA thread, issuing (not the tensor pipe, not L2) bounded the
        // kernel at ~1240 cycles per stage. The copies of stage s may start as soon as its bytes have
        // landed: full_bar[s] completing also means the MMAs that read the previous contents of this
        // stage's tensor-memory columns have retired (the producer waited for them).
        if (lane == 0) {
            const int which = warp - kFirstSfWarp;  // 0 tokens, 1 gate, 2 up
            constexpr uint32_t kStage16 = kStageBytes >> 4;
            const uint32_t sf_lo0 = umma_desc_lo_sf(smem_u32(smem + kABytes + kBBytes)) + which * (kSfBytes >> 4);
            const uint32_t col0 = which == 0 ? 0u : (which == 1 ? 16u : 20u);
            const uint32_t col_step = which == 0 ? 4u : 8u;
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < total_tiles && ok; item += gridDim.x) {
                for (int ks = 0; ks < k_stages; ++ks) {
                    if (!mbar_wait(&full_bar[s], ph, abort_flag, a.status, XMOE_DEV_TIMEOUT_TMA)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sf_lo = sf_lo0 + s * kStage16;
                    const uint32_t sf_tmem = tmem_base + kAccCols + s * kSfSlotCols + col0;
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) tmem_cp_sf_lo(sf_tmem + kb * col_step, sf_lo + kb * 32);
                    tc_commit(&sf_ready[s]);
                    if (++s == (uint32_t)kStages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else {
        // 8 epilogue warps: two per lane quadrant, each draining half of the 128 I columns, so
        // every scheduler has two warps to interleave around the transcendental unit.
        const int q = warp & 3;
        const int col_half = (warp - 2) >> 2;
        const float xgs_inv = a.scale->xgs_inv;
        uint16_t* yact = reinterpret_cast<uint16_t*>(a.yact);
        const uint16_t* row_w = reinterpret_cast<const uint16_t*>(a.row_weight);
        uint32_t tile_n = 0;
        for (int item = blockIdx.x; item < total_tiles; item += gridDim.x, ++tile_n) {
            const TileInfo t = tile_decode(item, prefix, a.counts, a.offsets, a.E_tot, kTokTile);
            const int n_local = q * 32 + lane;
            const bool row_ok = t.nt_idx * kTokTile + n_local < t.count;
            const int r = t.row0 + n_local;
            const float w = row_ok ? bf16_bits_to_f32(row_w[r]) : 0.f;
            const float sg = __fmul_rn(a.w13_gs[t.e * 2 + 0], xgs_inv);
            const float su = __fmul_rn(__fmul_rn(a.w13_gs[t.e * 2 + 1], xgs_inv), w);  // routing weight folded into the up scale
            const int i0 = t.wt * kWTile + col_half * 64;
            if (!mbar_wait(acc_full, tile_n & 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_ACC)) break;
            tc_fence_after();
            if (threadIdx.x == 64) XMOE_TRACE_STAMP(tile_n, 2);
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + col_half * 64;
#pragma unroll 1
            for (int c0 = 0; c0 < 64; c0 += 32) {
                if (i0 + c0 >= a.I) break;
                uint32_t g[32], u[32];
                tmem_ld32(lane_addr + c0, g);
                tmem_ld32(lane_addr + kWTile + c0, u);
                tmem_ld_wait();
                if (row_ok) {
                    uint32_t o[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float y0 = glu_apply(ACT, __uint_as_float(g[2 * j]), __uint_as_float(u[2 * j]), sg, su,
                                                   a.alpha, a.limit, w);
                        const float y1 = glu_apply(ACT, __uint_as_float(g[2 * j + 1]), __uint_as_float(u[2 * j + 1]), sg,
                                                   su, a.alpha, a.limit, w);
                        o[j] = pack_bf16x2(y0, y1);
                    }
                    uint4* dst = reinterpret_cast<uint4*>(yact + (size_t)r * a.I + i0 + c0);
#pragma unroll
                    for (int v = 0; v < 4; ++v)
                        if (i0 + c0 + v * 8 < a.I) dst[v] = make_uint4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (threadIdx.x == 64) XMOE_TRACE_STAMP(tile_n, 3);
            if (lane == 0) mbar_arrive(acc_empty);
        }
    }

    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

template <int ACT>
int launch_prefill_act(const Ff1Args& a, cudaStream_t stream) {
    static bool attr_set_dev[kMaxDevices] = {};
    const int dev = device_slot();
    if (dev < 0) return XMOE_ERR_CUDA;
    bool& attr_set = attr_set_dev[dev];
    if (!attr_set) {
        if (cudaFuncSetAttribute(ff1_nvfp4_prefill_kernel<ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kSmemBytes) != cudaSuccess)
            return XMOE_ERR_CUDA;
        attr_set = true;
    }
    ff1_nvfp4_prefill_kernel<ACT><<<a.num_sms, kThreads, kSmemBytes, stream>>>(a);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

}  // namespace

#ifdef XMOE_TRACE
extern "C" int xmoe_ff1_trace_dump(unsigned long long* host_out) {
    return (int)cudaMemcpyFromSymbol(host_out, g_ff1_trace, sizeof(g_ff1_trace));
}
#endif

int launch_ff1_prefill(const Ff1Args& a, cudaStream_t stream) {
    switch (a.activation) {
        case 0: return launch_prefill_act<0>(a, stream);
        case 1: return launch_prefill_act<1>(a, stream);
        case 2: return launch_prefill_act<2>(a, stream);
        default: return XMOE_ERR_SHAPE;
    }
}

}  // namespace xmoe
