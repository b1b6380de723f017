// FF1: grouped NVFP4 W4A4 gate/up GEMM with a fused SwiGLU * routing-weight epilogue.
//
// Math follows the reference FF1 (xFused-NVFP4-Kernels/xMoE/xW4A16/sm120a/xR64FF1FF2/
// xR64FF1.cu:65-651 and co-design.md:75-90): G = W1 x, U = W3 x with fp32 accumulation
// over NVFP4 x NVFP4 products, both scaled by weight_global_scale * act_inverse_scale,
// silu(G) * U in fp32, times the routing weight, rounded to bf16. The weight tensors keep
// the checkpoint layout the reference documents at xR64FF1.cu:17-20
// (W13 u8 [E, 2I, H/2], low nibble = lower K). The intermediate stays bf16 because the
// down projection here is W4A16.
//
// B200 design (nothing of the reference's mma.sync structure is kept):
//   * swap-AB: 128 weight rows are the MMA M operand, NT tokens the N operand, so decode
//     batches do not pad to 128 rows; gate and up tiles of the same I-range accumulate
//     into two TMEM accumulators and meet in the same epilogue thread (TMEM lane = I row).
//   * persistent CTAs, one per SM, walk a tile list (expert, I-tile, token-tile) derived
//     on the device from the expert histogram.
//   * warp 0 issues TMA (2-D tiled loads with the 128-byte swizzle for W and X, bulk
//     copies for the pre-ordered scale factors) into a multi-stage ring; warp 1 copies the
//     scale factors into TMEM (tcgen05.cp) and issues tcgen05.mma kind::mxf4nvf4
//     (K = 64 per instruction, 4 per stage); warps 2-5 drain the accumulators with
//     tcgen05.ld and run the epilogue.
//   * every mbarrier wait is bounded; on a timeout the CTA flags the status word and
//     all roles fall through to the common exit, where TMEM is released.
#include "common.cuh"
#include "kernels.h"
#include "tile_sched.cuh"

namespace xmoe {

namespace {

constexpr int kBlockM = 128;          // weight rows per tile (per projection)
constexpr int kStageKBytes = 128;     // packed bytes along K per stage = 256 K elements
constexpr int kKPerStage = 256;
constexpr int kSfStageBytes = 2048;   // 4 K-blocks of 64 x 512-byte scale tiles
constexpr int kThreads = 288;         // producer warp, MMA warp, 4 epilogue warps, 3 scale-factor copy warps
constexpr int kFirstSfWarp = 6;
constexpr int kMaxExperts = 1024 + 8;
constexpr int kTmemCols = 512;

template <int NT>
struct Ff1Cfg {
    static constexpr int kABytes = kBlockM * kStageKBytes;  // 16 KiB per projection
    static constexpr int kBBytes = NT * kStageKBytes;
    static constexpr int kStageBytes = 2 * kABytes + kBBytes + 3 * kSfStageBytes;
    static constexpr int kStages = NT >= 128 ? 4 : (NT >= 64 ? 4 : 5);
    static constexpr int kAccStages = NT >= 128 ? 1 : 2;
    static constexpr int kAccCols = 2 * NT;                 // gate + up
    static constexpr int kSfColsBase = kAccStages * kAccCols;
    static constexpr int kSfColsPerSlot = 48;               // 4 K-blocks x (gate 4 + up 4 + tokens 4)
    static_assert(kSfColsBase + kStages * kSfColsPerSlot <= kTmemCols, "TMEM budget");  // one slot per stage
    static constexpr int kTxBytes = kStageBytes;
    static constexpr size_t kSmemBytes = 1024 /*align slack*/ + (size_t)kStages * kStageBytes + 8192;
};

template <int NT>
__global__ __launch_bounds__(kThreads, 1) void ff1_nvfp4_kernel(const __grid_constant__ Ff1Args a) {
    using Cfg = Ff1Cfg<NT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* stage_base = smem;
    uint8_t* tail = smem + (size_t)Cfg::kStages * Cfg::kStageBytes;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);             // [kStages]
    uint64_t* empty_bar = full_bar + 8;                                 // [kStages]
    uint64_t* acc_full = empty_bar + 8;                                 // [2]
    uint64_t* acc_empty = acc_full + 2;                                 // [2]
    uint64_t* sf_ready = acc_empty + 2;                                 // [kStages] scale factors of the stage are in tensor memory
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sf_ready + 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    int* prefix = reinterpret_cast<int*>(tail + 256);                   // [e_tot + 1]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int mt_tiles = a.mb;
    const int k_stages = (a.H + kKPerStage - 1) / kKPerStage;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
            mbar_init(&sf_ready[s], 3);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 4);
        }
        *abort_flag = 0u;
        mbar_fence_init();
        prefetch_tmap(&a.tm_w);
        prefetch_tmap(&a.tm_x);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    if (warp == 2) tile_prefix_build(prefix, a.counts, a.E_tot, mt_tiles, NT);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int total_tiles = prefix[a.E_tot];
    const int tile_stride = balanced_stride(total_tiles, (int)gridDim.x);
    const int first_tile = (int)blockIdx.x < tile_stride ? (int)blockIdx.x : total_tiles;  // CTAs beyond the stride idle

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int item = first_tile; item < total_tiles && ok; item += tile_stride) {
                const TileInfo t = tile_decode(item, prefix, a.counts, a.offsets, a.E_tot, NT);
                const int gate_row = t.e * 2 * a.I + t.wt * kBlockM;
                const int up_row = gate_row + a.I;
                const uint8_t* sfw_g = a.sfw + ((size_t)(t.e * 2 + 0) * a.mb + t.wt) * a.kb_pad * 512;
                const uint8_t* sfw_u = a.sfw + ((size_t)(t.e * 2 + 1) * a.mb + t.wt) * a.kb_pad * 512;
                const uint8_t* sfx = a.sfx + (size_t)(t.row0 / NT) * a.kb_pad * 512;
                for (int ks = 0; ks < k_stages; ++ks, ++it) {
                    const int s = it % Cfg::kStages;
                    const uint32_t ph = (it / Cfg::kStages) & 1u;
                    if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_MMA)) {
                        ok = false;
                        break;
                    }
                    uint8_t* st = stage_base + (size_t)s * Cfg::kStageBytes;
                    mbar_expect_tx(&full_bar[s], Cfg::kTxBytes);
                    tma_load_2d(st, &a.tm_w, ks * kStageKBytes, gate_row, &full_bar[s]);
                    tma_load_2d(st + Cfg::kABytes, &a.tm_w, ks * kStageKBytes, up_row, &full_bar[s]);
                    tma_load_2d(st + 2 * Cfg::kABytes, &a.tm_x, ks * kStageKBytes, t.row0, &full_bar[s]);
                    uint8_t* sf = st + 2 * Cfg::kABytes + Cfg::kBBytes;
                    tma_load_1d(sf, sfw_g + (size_t)ks * kSfStageBytes, kSfStageBytes, &full_bar[s]);
                    tma_load_1d(sf + kSfStageBytes, sfw_u + (size_t)ks * kSfStageBytes, kSfStageBytes, &full_bar[s]);
                    tma_load_1d(sf + 2 * kSfStageBytes, sfx + (size_t)ks * kSfStageBytes, kSfStageBytes, &full_bar[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_nvfp4(kBlockM, NT);
            constexpr uint32_t kStage16 = Cfg::kStageBytes >> 4;
            const uint32_t ag_lo0 = umma_desc_lo_sw128(smem_u32(stage_base));
            const uint32_t au_lo0 = umma_desc_lo_sw128(smem_u32(stage_base + Cfg::kABytes));
            const uint32_t b_lo0 = umma_desc_lo_sw128(smem_u32(stage_base + 2 * Cfg::kABytes));
            uint32_t tile_n = 0, s = 0, ph = 0;
            bool ok = true;
            for (int item = first_tile; item < total_tiles && ok; item += tile_stride, ++tile_n) {
                const uint32_t as = tile_n % Cfg::kAccStages;
                const uint32_t aph = (tile_n / Cfg::kAccStages) & 1u;
                if (!mbar_wait(&acc_empty[as], aph ^ 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_EPI)) break;
                tc_fence_after();
                const uint32_t acc_gate = tmem_base + as * Cfg::kAccCols;
                const uint32_t acc_up = acc_gate + NT;
                for (int ks = 0; ks < k_stages; ++ks) {
                    if (!mbar_wait(&full_bar[s], ph, abort_flag, a.status, XMOE_DEV_TIMEOUT_TMA) ||
                        !mbar_wait(&sf_ready[s], ph, abort_flag, a.status, XMOE_DEV_TIMEOUT_TMA)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sf_tmem = tmem_base + Cfg::kSfColsBase + s * Cfg::kSfColsPerSlot;
                    const uint32_t ag_lo = ag_lo0 + s * kStage16, au_lo = au_lo0 + s * kStage16;
                    const uint32_t b_lo = b_lo0 + s * kStage16;
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) {
                        const uint32_t acc = (ks | kb) ? 1u : 0u;  // 32 bytes of packed K per MMA: +2 descriptor units
                        mma_nvfp4_lo(acc_gate, ag_lo + kb * 2, b_lo + kb * 2, idesc, sf_tmem + kb * 4,
                                     sf_tmem + 32 + kb * 4, acc);
                        mma_nvfp4_lo(acc_up, au_lo + kb * 2, b_lo + kb * 2, idesc, sf_tmem + 16 + kb * 4,
                                     sf_tmem + 32 + kb * 4, acc);
                    }
                    tc_commit(&empty_bar[s]);
                    if (++s == (uint32_t)Cfg::kStages) { s = 0; ph ^= 1u; }
                }
                if (ok) tc_commit(&acc_full[as]);
            }
        }
    } else if (warp >= kFirstSfWarp) {
        // ------------------------------ scale-factor copies ------------------------
        // One thread per operand (gate rows, up rows, tokens) moves the stage's scale factors from
        // shared to tensor memory. A thread issues one tcgen05 instruction per ~65 cycles: with these
        // 12 copies on the MMA thread (21 instructions per 40 KB stage) issuing capped the kernel
        // near 8 TB/s. full_bar[s] completing also means the MMAs that read the previous contents of
        // this stage's tensor-memory columns have retired (the producer waited for them).
        if (lane == 0) {
            const int which = warp - kFirstSfWarp;  // 0 gate, 1 up, 2 tokens
            constexpr uint32_t kStage16 = Cfg::kStageBytes >> 4;
            const uint32_t sf_lo0 = umma_desc_lo_sf(smem_u32(stage_base + 2 * Cfg::kABytes + Cfg::kBBytes)) +
                                    which * (kSfStageBytes >> 4);
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (int item = first_tile; item < total_tiles && ok; item += tile_stride) {
                for (int ks = 0; ks < k_stages; ++ks) {
                    if (!mbar_wait(&full_bar[s], ph, abort_flag, a.status, XMOE_DEV_TIMEOUT_TMA)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sf_lo = sf_lo0 + s * kStage16;
                    const uint32_t sf_tmem = tmem_base + Cfg::kSfColsBase + s * Cfg::kSfColsPerSlot + which * 16;
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) tmem_cp_sf_lo(sf_tmem + kb * 4, sf_lo + kb * 32);
                    tc_commit(&sf_ready[s]);
                    if (++s == (uint32_t)Cfg::kStages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else {
        // ------------------------------ epilogue -----------------------------------
        const int q = warp & 3;  // TMEM lane quadrant this warp may read
        const float xgs_inv = a.scale->xgs_inv;
        uint32_t tile_n = 0;
        uint16_t* yact = reinterpret_cast<uint16_t*>(a.yact);
        const uint16_t* row_w = reinterpret_cast<const uint16_t*>(a.row_weight);
        for (int item = first_tile; item < total_tiles; item += tile_stride, ++tile_n) {
            const TileInfo t = tile_decode(item, prefix, a.counts, a.offsets, a.E_tot, NT);
            const uint32_t as = tile_n % Cfg::kAccStages;
            const uint32_t aph = (tile_n / Cfg::kAccStages) & 1u;
            if (!mbar_wait(&acc_full[as], aph, abort_flag, a.status, XMOE_DEV_TIMEOUT_ACC)) break;
            tc_fence_after();
            const float sg = __fmul_rn(a.w13_gs[t.e * 2 + 0], xgs_inv);
            const float su = __fmul_rn(a.w13_gs[t.e * 2 + 1], xgs_inv);
            const int i_idx = t.wt * kBlockM + q * 32 + lane;
            const bool i_ok = i_idx < a.I;
            const int n_valid = min(NT, t.count - t.nt_idx * NT);
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + as * Cfg::kAccCols;
            for (int c0 = 0; c0 < NT; c0 += 32) {
                if (c0 >= n_valid) break;
                uint32_t g[32], u[32];
                tmem_ld32(lane_addr + c0, g);
                tmem_ld32(lane_addr + NT + c0, u);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int n = c0 + j;
                    if (n < n_valid && i_ok) {
                        const int r = t.row0 + n;
                        const float w = bf16_bits_to_f32(row_w[r]);
                        const float y = glu_apply(a.activation, __uint_as_float(g[j]), __uint_as_float(u[j]), sg,
                                                  __fmul_rn(su, w), a.alpha, a.limit, w);
                        yact[(size_t)r * a.I + i_idx] = (uint16_t)f32_to_bf16_bits(y);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[as]);
        }
    }

    // common exit: after an abort give in-flight copies / MMAs a bounded moment to land
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

template <int NT>
int launch_ff1_nt(const Ff1Args& a, cudaStream_t stream) {
    using Cfg = Ff1Cfg<NT>;
    static bool attr_set_dev[kMaxDevices] = {};
    const int dev = device_slot();
    if (dev < 0) return XMOE_ERR_CUDA;
    bool& attr_set = attr_set_dev[dev];
    if (!attr_set) {
        if (cudaFuncSetAttribute(ff1_nvfp4_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)Cfg::kSmemBytes) != cudaSuccess)
            return XMOE_ERR_CUDA;
        attr_set = true;
    }
    ff1_nvfp4_kernel<NT><<<a.num_sms, kThreads, Cfg::kSmemBytes, stream>>>(a);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

}  // namespace

int launch_ff1(const Ff1Args& a, cudaStream_t stream) {
    if (a.E_tot + 1 > kMaxExperts || a.H % 64 || a.I % 16) return XMOE_ERR_SHAPE;
    switch (a.nt) {
        case 32: return launch_ff1_nt<32>(a, stream);
        case 64: return launch_ff1_nt<64>(a, stream);
        case 128: return launch_ff1_prefill(a, stream);  // token-major variant, ff1_nvfp4_prefill.cu
        default: return XMOE_ERR_SHAPE;
    }
}

}  // namespace xmoe
