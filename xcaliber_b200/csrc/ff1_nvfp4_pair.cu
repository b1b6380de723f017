// FF1 for prefill on CTA PAIRS: the token-major NVFP4 gate/up GEMM of ff1_nvfp4_prefill.cu
// (same math, same epilogue, reference pointers there) issued as 2-SM MMAs
// (tcgen05 cta_group::2, M = 256 tokens, N = 256 = 128 gate | 128 up rows, K = 64).
//
// Why: a single CTA stages 54 KB per 16.8 MFLOP and the kernel ran at what the L2 -> SM path
// delivers (~9 TB/s => ~2.9 PFLOP/s). In a pair each CTA stages its own 128 token rows and only
// HALF of the weight tile: the leader the 128 gate rows, the peer the 128 up rows. The MMA reads
// both halves, every CTA gets gate and up columns for its own 128 tokens, and weight traffic
// per SM halves (38 KB per 16.8 MFLOP).
//
// The epilogue warps hold their whole accumulator slice in registers (setmaxnreg moves registers to
// them from the single-thread roles) and release the accumulator right after copying it: SwiGLU and
// the stores of tile t overlap the MMAs of tile t + 1 (un-overlapped, the epilogue was 27 % of the
// kernel). What bounds the kernel now is L2 -> SM delivery of 38 KB per K 256 stage.
//
// Scale factors: each CTA needs the token scales of its own rows and the weight scales of ALL 256
// N rows in its tensor memory, so both CTAs load both (2 KB each per stage). Three threads of the
// leader (tokens / gate / up) issue the cta_group::2 tcgen05.cp that copy from each CTA's shared
// memory into that CTA's tensor memory; the MMA thread only waits, issues four MMAs and two commits
// per stage (a thread issues one tcgen05 instruction per ~65 cycles: with the copies on the MMA
// thread the kernel was issue-bound). Cross-CTA protocol: the peer's relay thread reports a landed
// stage with a remote arrive on the leader's full barrier (count 2: own bytes + the report); the
// leader's commits carry an arrival mask and release the stage / accumulator barriers of both
// CTAs; both epilogues report to the leader. No data multicast; every wait is bounded.
#include <cstdio>
#include <cstdlib>

#include "cluster.cuh"
#include "common.cuh"
#include "kernels.h"
#include "tile_sched.cuh"

namespace xmoe {

#ifdef XMOE_TRACE
__device__ long long g_ff1p_trace[148 * 8];
#define XMOE_T0() const long long t0__ = clock64()
#define XMOE_TACC(var) var += clock64() - t0__
#else
#define XMOE_T0() do {} while (0)
#define XMOE_TACC(var) do {} while (0)
#endif

namespace {

constexpr int kTokHalf = 128;          // token rows per CTA
constexpr int kTokTile = 256;          // token rows per pair tile
constexpr int kWTile = 128;            // I rows per tile (per projection)
constexpr int kStageKBytes = 128;      // 256 K elements per stage
constexpr int kKPerStage = 256;
constexpr int kSfBytes = 2048;
constexpr int kABytes = kTokHalf * kStageKBytes;   // 16 KiB: my tokens
constexpr int kBBytes = kWTile * kStageKBytes;     // 16 KiB: my half of the weight tile
constexpr int kStageBytes = kABytes + kBBytes + 3 * kSfBytes;  // 38 KiB
constexpr int kStages = 5;
#ifndef XMOE_FF1_PRODUCERS
#define XMOE_FF1_PRODUCERS 2
#endif
constexpr int kProducers = XMOE_FF1_PRODUCERS;  // 2: tokens and weights are requested by different threads
constexpr int kWeightProducerWarp = 13;
// Warp roles, arranged so that register reallocation (setmaxnreg, per group of 4 consecutive warps)
// can move registers from the single-thread roles to the epilogue:
//   warps 0-3  : TMA producer, MMA issuer (peer: relay), scale-factor copies of tokens / gate rows
//   warps 4-11 : epilogue (two per tensor-memory lane quadrant)
//   warp 12    : scale-factor copies of the up rows; warps 13-15 idle
constexpr int kThreads = 512;
constexpr int kFirstEpiWarp = 4;
constexpr int kLastSfWarp = 12;
constexpr int kRegsFew = 40;    // single-thread roles
constexpr int kRegsEpi = 208;   // epilogue: 128 accumulator values in flight per thread
static_assert(2 * 128 * (kRegsEpi - 128) <= 2 * 128 * (128 - kRegsFew), "register pool: 512 threads x 128 at launch");
constexpr int kTmemCols = 512;
constexpr int kAccCols = 256;
constexpr int kSfSlotCols = 48;
static_assert(kAccCols + kStages * kSfSlotCols <= kTmemCols, "TMEM budget");
constexpr size_t kSmemBytes = 1024 + (size_t)kStages * kStageBytes + 8192;

template <int ACT>
__global__ __launch_bounds__(kThreads, 1) void ff1_nvfp4_pair_kernel(const __grid_constant__ Ff1Args a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* tail = smem + (size_t)kStages * kStageBytes;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);  // [8] local: my stage landed
    uint64_t* sf_ready = full_bar + 8;                       // [8] leader: the stage's scale factors are in both CTAs' tensor memory
    uint64_t* empty_bar = sf_ready + 8;                      // [8] each CTA: MMAs reading the stage retired
    uint64_t* acc_full = empty_bar + 8;                      // [1] each CTA
    uint64_t* acc_empty = acc_full + 1;                      // [1] leader: 16 epilogue warps drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    int* prefix = reinterpret_cast<int*>(tail + 256);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int cluster_id = blockIdx.x >> 1;
    const int n_clusters = gridDim.x >> 1;
    const int w_tiles = a.mb;
    const int k_stages = (a.H + kKPerStage - 1) / kKPerStage;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            // one arrival per producer thread of this CTA; leader: + the peer's report that its stage landed
            mbar_init(&full_bar[s], kProducers + (leader ? 1 : 0));
            mbar_init(&sf_ready[s], 3);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 16);
        *abort_flag = 0u;
        mbar_fence_init();
        prefetch_tmap(&a.tm_w);
        prefetch_tmap(&a.tm_x);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, kTmemCols);
        tmem_relinquish_pair();
    }
    if (warp == 2) tile_prefix_build(prefix, a.counts, a.E_tot, w_tiles, kTokTile);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int total_tiles = prefix[a.E_tot];

    // Register reallocation by groups of four warps (all threads of a group take the same branch): the
    // epilogue keeps a whole accumulator slice in registers so that it can hand the accumulator back
    // before doing its arithmetic and stores; the single-thread roles give their registers up.
    if (warp >= kFirstEpiWarp && warp < kFirstEpiWarp + 8) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsEpi));
        // ---- epilogue: my 128 tokens x (128 gate | 128 up) columns, 8 warps. Each warp first copies its
        // whole slice (64 gate + 64 up columns) to registers and releases the accumulator: the next tile's
        // MMAs run while this one's SwiGLU and stores are done (the un-overlapped epilogue was 27 % of
        // the kernel).
        const int q = warp & 3;
        const int col_half = (warp - kFirstEpiWarp) >> 2;
        const float xgs_inv = a.scale->xgs_inv;
        uint16_t* yact = reinterpret_cast<uint16_t*>(a.yact);
        const uint16_t* row_w = reinterpret_cast<const uint16_t*>(a.row_weight);
        const uint32_t leader_acc_empty = map_to_cta(smem_u32(acc_empty), 0);
        uint32_t tile_n = 0;
        for (int item = cluster_id; item < total_tiles; item += n_clusters, ++tile_n) {
            const TileInfo t = tile_decode(item, prefix, a.counts, a.offsets, a.E_tot, kTokTile);
            const int n_local = (int)rank * kTokHalf + q * 32 + lane;
            const bool row_ok = t.nt_idx * kTokTile + n_local < t.count;
            const int r = t.row0 + n_local;
            const float w = row_ok ? bf16_bits_to_f32(row_w[r]) : 0.f;
            const float sg = __fmul_rn(a.w13_gs[t.e * 2 + 0], xgs_inv);
            const float su = __fmul_rn(__fmul_rn(a.w13_gs[t.e * 2 + 1], xgs_inv), w);
            const int i0 = t.wt * kWTile + col_half * 64;
            if (!mbar_wait_cluster(acc_full, tile_n & 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_ACC)) break;
            tc_fence_after();
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + col_half * 64;
            uint32_t g[64], u[64];
            tmem_ld32(lane_addr, g);
            tmem_ld32(lane_addr + 32, g + 32);
            tmem_ld32(lane_addr + kWTile, u);
            tmem_ld32(lane_addr + kWTile + 32, u + 32);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_acc_empty);  // the accumulator is free again
            if (row_ok) {
#pragma unroll
                for (int c0 = 0; c0 < 64; c0 += 32) {
                    if (i0 + c0 < a.I) {
                        uint32_t o[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float y0 = glu_apply(ACT, __uint_as_float(g[c0 + 2 * j]), __uint_as_float(u[c0 + 2 * j]),
                                                       sg, su, a.alpha, a.limit, w);
                            const float y1 = glu_apply(ACT, __uint_as_float(g[c0 + 2 * j + 1]),
                                                       __uint_as_float(u[c0 + 2 * j + 1]), sg, su, a.alpha, a.limit, w);
                            o[j] = pack_bf16x2(y0, y1);
                        }
                        uint4* dst = reinterpret_cast<uint4*>(yact + (size_t)r * a.I + i0 + c0);
#pragma unroll
                        for (int v = 0; v < 4; ++v)
                            if (i0 + c0 + v * 8 < a.I) dst[v] = make_uint4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
                    }
                }
            }
        }
    } else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsFew));
        if (warp == 0) {
            // ---- producer: my 128 tokens, my half of the weight tile, all scale factors ----
            if (lane == 0) {
                uint32_t s = 0, ph = 0;
                bool ok = true;
                for (int item = cluster_id; item < total_tiles && ok; item += n_clusters) {
                    const TileInfo t = tile_decode(item, prefix, a.counts, a.offsets, a.E_tot, kTokTile);
                    const int tok_row = t.row0 + (int)rank * kTokHalf;
                    const int w_row = t.e * 2 * a.I + (int)rank * a.I + t.wt * kWTile;  // leader: gate rows, peer: up rows
                    const uint8_t* sfw_g = a.sfw + ((size_t)(t.e * 2 + 0) * a.mb + t.wt) * a.kb_pad * 512;
                    const uint8_t* sfw_u = a.sfw + ((size_t)(t.e * 2 + 1) * a.mb + t.wt) * a.kb_pad * 512;
                    const uint8_t* sfx = a.sfx + (size_t)(tok_row / kTokHalf) * a.kb_pad * 512;
                    for (int ks = 0; ks < k_stages; ++ks) {
                        if (!mbar_wait_cluster(&empty_bar[s], ph ^ 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_MMA)) {
                            ok = false;
                            break;
                        }
                        uint8_t* st = smem + (size_t)s * kStageBytes;
                        uint8_t* sf = st + kABytes + kBBytes;
                        if (kProducers == 1) {
                            mbar_expect_tx(&full_bar[s], kStageBytes);
                            tma_load_2d(st, &a.tm_x, ks * kStageKBytes, tok_row, &full_bar[s]);
                            tma_load_2d(st + kABytes, &a.tm_w, ks * kStageKBytes, w_row, &full_bar[s]);
                            tma_load_1d(sf, sfx + (size_t)ks * kSfBytes, kSfBytes, &full_bar[s]);
                            tma_load_1d(sf + kSfBytes, sfw_g + (size_t)ks * kSfBytes, kSfBytes, &full_bar[s]);
                            tma_load_1d(sf + 2 * kSfBytes, sfw_u + (size_t)ks * kSfBytes, kSfBytes, &full_bar[s]);
                        } else {  // this thread: my tokens and their scale factors
                            mbar_expect_tx(&full_bar[s], kABytes + kSfBytes);
                            tma_load_2d(st, &a.tm_x, ks * kStageKBytes, tok_row, &full_bar[s]);
                            tma_load_1d(sf, sfx + (size_t)ks * kSfBytes, kSfBytes, &full_bar[s]);
                        }
                        if (++s == (uint32_t)kStages) { s = 0; ph ^= 1u; }
                    }
                }
            }
        } else if (warp == 1) {
            if (lane == 0 && leader) {
                // ---- MMA issuer (leader) ----
                constexpr uint32_t idesc = umma_idesc_nvfp4(2 * kTokHalf, 2 * kWTile);
                constexpr uint32_t kStage16 = kStageBytes >> 4;
                const uint32_t a_lo0 = umma_desc_lo_sw128(smem_u32(smem));
                const uint32_t b_lo0 = umma_desc_lo_sw128(smem_u32(smem + kABytes));
                uint32_t tile_n = 0, s = 0, ph = 0;
                bool ok = true;
                long long tw_acc = 0, tw_full = 0, tw_sf = 0, t_issue = 0;
                (void)tw_acc; (void)tw_full; (void)tw_sf; (void)t_issue;
                const long long t_start = clock64();
                (void)t_start;
                for (int item = cluster_id; item < total_tiles && ok; item += n_clusters, ++tile_n) {
                    {
                        XMOE_T0();
                        if (!mbar_wait_cluster(acc_empty, (tile_n & 1u) ^ 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_EPI)) break;
                        XMOE_TACC(tw_acc);
                    }
                    tc_fence_after();
                    for (int ks = 0; ks < k_stages; ++ks) {
                        {
                            XMOE_T0();
                            if (!mbar_wait_cluster(&full_bar[s], ph, abort_flag, a.status, XMOE_DEV_TIMEOUT_TMA)) { ok = false; break; }
                            XMOE_TACC(tw_full);
                        }
                        {
                            XMOE_T0();
                            if (!mbar_wait(&sf_ready[s], ph, abort_flag, a.status, XMOE_DEV_TIMEOUT_TMA)) { ok = false; break; }
                            XMOE_TACC(tw_sf);
                        }
                        XMOE_T0();
                        tc_fence_after();
                        const uint32_t sf_tmem = tmem_base + kAccCols + s * kSfSlotCols;
                        const uint32_t a_lo = a_lo0 + s * kStage16;
                        const uint32_t b_lo = b_lo0 + s * kStage16;
    #pragma unroll
                        for (int kb = 0; kb < 4; ++kb)
                            mma_nvfp4_pair(tmem_base, a_lo + kb * 2, b_lo + kb * 2, idesc, sf_tmem + kb * 4,
                                           sf_tmem + 16 + kb * 8, (ks | kb) ? 1u : 0u);
                        tc_commit_pair_mask(smem_u32(&empty_bar[s]), 3);
                        if (++s == (uint32_t)kStages) { s = 0; ph ^= 1u; }
                        XMOE_TACC(t_issue);
                    }
                    if (ok) tc_commit_pair_mask(smem_u32(acc_full), 3);
                }
    #ifdef XMOE_TRACE
                if (cluster_id < 148) {
                    long long* o = g_ff1p_trace + cluster_id * 8;
                    o[0] = tw_full; o[1] = tw_sf; o[2] = tw_acc; o[3] = t_issue; o[4] = clock64() - t_start; o[5] = tile_n;
                }
    #endif
            } else if (lane == 0) {
                // ---- relay (peer): report landed stages to the leader ----
                const uint32_t leader_full = map_to_cta(smem_u32(&full_bar[0]), 0);
                uint32_t s = 0, ph = 0;
                bool ok = true;
                for (int item = cluster_id; item < total_tiles && ok; item += n_clusters) {
                    for (int ks = 0; ks < k_stages; ++ks) {
                        if (!mbar_wait(&full_bar[s], ph, abort_flag, a.status, XMOE_DEV_TIMEOUT_TMA)) {
                            ok = false;
                            break;
                        }
                        mbar_arrive_cluster(leader_full + s * 8u);
                        if (++s == (uint32_t)kStages) { s = 0; ph ^= 1u; }
                    }
                }
            }
        } else if (kProducers == 2 && warp == kWeightProducerWarp) {
            // ---- second producer: my half of the weight tile and the weight scale factors of both halves ----
            if (lane == 0) {
                uint32_t s = 0, ph = 0;
                bool ok = true;
                for (int item = cluster_id; item < total_tiles && ok; item += n_clusters) {
                    const TileInfo t = tile_decode(item, prefix, a.counts, a.offsets, a.E_tot, kTokTile);
                    const int w_row = t.e * 2 * a.I + (int)rank * a.I + t.wt * kWTile;  // leader: gate rows, peer: up rows
                    const uint8_t* sfw_g = a.sfw + ((size_t)(t.e * 2 + 0) * a.mb + t.wt) * a.kb_pad * 512;
                    const uint8_t* sfw_u = a.sfw + ((size_t)(t.e * 2 + 1) * a.mb + t.wt) * a.kb_pad * 512;
                    for (int ks = 0; ks < k_stages; ++ks) {
                        if (!mbar_wait_cluster(&empty_bar[s], ph ^ 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_MMA)) {
                            ok = false;
                            break;
                        }
                        uint8_t* st = smem + (size_t)s * kStageBytes;
                        uint8_t* sf = st + kABytes + kBBytes;
#ifdef XMOE_FF1_EXPERIMENT_SKIP_SFU  // timing experiment only (wrong results): one request fewer per stage
                        mbar_expect_tx(&full_bar[s], kBBytes + kSfBytes);
                        tma_load_2d(st + kABytes, &a.tm_w, ks * kStageKBytes, w_row, &full_bar[s]);
                        tma_load_1d(sf + kSfBytes, sfw_g + (size_t)ks * kSfBytes, kSfBytes, &full_bar[s]);
                        (void)sfw_u;
#else
                        mbar_expect_tx(&full_bar[s], kBBytes + 2 * kSfBytes);
                        tma_load_2d(st + kABytes, &a.tm_w, ks * kStageKBytes, w_row, &full_bar[s]);
                        tma_load_1d(sf + kSfBytes, sfw_g + (size_t)ks * kSfBytes, kSfBytes, &full_bar[s]);
                        tma_load_1d(sf + 2 * kSfBytes, sfw_u + (size_t)ks * kSfBytes, kSfBytes, &full_bar[s]);
#endif
                        if (++s == (uint32_t)kStages) { s = 0; ph ^= 1u; }
                    }
                }
            }
        } else if (warp == 2 || warp == 3 || warp == kLastSfWarp) {
            // ---- scale-factor copies (leader): one thread per operand; a cta_group::2 copy moves each
            // CTA's shared-memory tile into that CTA's tensor memory. A stage's copies may start once
            // BOTH CTAs' bytes have landed (the leader's full barrier counts the peer's report).
            if (lane == 0 && leader) {
                const int which = warp == kLastSfWarp ? 2 : warp - 2;  // 0 my tokens, 1 gate rows, 2 up rows
                constexpr uint32_t kStage16 = kStageBytes >> 4;
                const uint32_t sf_lo0 = umma_desc_lo_sf(smem_u32(smem + kABytes + kBBytes)) + which * (kSfBytes >> 4);
                const uint32_t col0 = which == 0 ? 0u : (which == 1 ? 16u : 20u);
                const uint32_t col_step = which == 0 ? 4u : 8u;
                uint32_t s = 0, ph = 0;
                bool ok = true;
                for (int item = cluster_id; item < total_tiles && ok; item += n_clusters) {
                    for (int ks = 0; ks < k_stages; ++ks) {
                        if (!mbar_wait_cluster(&full_bar[s], ph, abort_flag, a.status, XMOE_DEV_TIMEOUT_TMA)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        const uint32_t sf_lo = sf_lo0 + s * kStage16;
                        const uint32_t sf_tmem = tmem_base + kAccCols + s * kSfSlotCols + col0;
    #pragma unroll
                        for (int kb = 0; kb < 4; ++kb) tmem_cp_sf_pair(sf_tmem + kb * col_step, sf_lo + kb * 32);
                        tc_commit_pair(smem_u32(&sf_ready[s]));
                        if (++s == (uint32_t)kStages) { s = 0; ph ^= 1u; }
                    }
                }
            }
        }
    }

    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    cluster_sync_all();
    if (warp == 1) tmem_dealloc_pair(tmem_base, kTmemCols);
}

template <int ACT>
int launch_pair_act(const Ff1Args& a, cudaStream_t stream) {
    static bool attr_set_dev[kMaxDevices] = {};
    const int dev = device_slot();
    if (dev < 0) return XMOE_ERR_CUDA;
    bool& attr_set = attr_set_dev[dev];
    if (!attr_set) {
        if (cudaFuncSetAttribute(ff1_nvfp4_pair_kernel<ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kSmemBytes) != cudaSuccess)
            return XMOE_ERR_CUDA;
        attr_set = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(a.num_sms & ~1), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // Persistent kernel: launch exactly as many clusters as can be resident at once. Pairs must sit
    // inside one GPC, so this can be fewer than num_sms / 2; extra clusters would run as a second
    // wave and double the kernel time.
    static int resident_clusters_dev[kMaxDevices] = {};
    int& resident_clusters = resident_clusters_dev[dev];
    if (!resident_clusters) {
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, ff1_nvfp4_pair_kernel<ACT>, &cfg) != cudaSuccess || n <= 0) n = a.num_sms / 2;
        resident_clusters = n < a.num_sms / 2 ? n : a.num_sms / 2;
        if (getenv("XMOE_DEBUG"))
            fprintf(stderr, "xmoe: ff1 pair kernel: %d resident clusters of 2 CTAs (occupancy query %d, %d SMs)\n",
                    resident_clusters, n, a.num_sms);
    }
    cfg.gridDim = dim3((unsigned)(2 * resident_clusters), 1, 1);
    return cudaLaunchKernelEx(&cfg, ff1_nvfp4_pair_kernel<ACT>, a) == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

}  // namespace

#ifdef XMOE_TRACE
extern "C" int xmoe_ff1_pair_trace_dump(long long* host_out) {
    return (int)cudaMemcpyFromSymbol(host_out, g_ff1p_trace, sizeof(g_ff1p_trace));
}
#endif

int launch_ff1_pair(const Ff1Args& a, cudaStream_t stream) {
    switch (a.activation) {
        case 0: return launch_pair_act<0>(a, stream);
        case 1: return launch_pair_act<1>(a, stream);
        case 2: return launch_pair_act<2>(a, stream);
        default: return XMOE_ERR_SHAPE;
    }
}

}  // namespace xmoe
