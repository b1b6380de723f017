// FF2 for long-K prefill on CTA PAIRS: the same W4A16 down projection as ff2_w4a16.cu (weight
// contract, expansion arithmetic and tensor-memory A operand are identical; reference pointers
// are listed there), issued as 2-SM MMAs (tcgen05 cta_group::2, M = 256, N = 256).
//
// Why: with 128 weight rows per tile the 256-token activation tile is re-read from L2 once per
// 128 output features, and at ~9 TB/s of L2 delivery that capped the single-CTA kernel near
// 1.0 PFLOP/s. A cluster of two CTAs works on 256 weight rows: each CTA stages only HALF of the
// token tile (128 rows), expands its own 128 weight rows into its own tensor memory, and the
// leader CTA issues one MMA per K16 that reads both halves. Token-tile traffic per SM halves.
//
// Cross-CTA protocol (no data multicast anywhere; plain TMA loads with local barriers):
//   * peer -> leader: "my half of the token stage landed" (relay thread, remote arrive on the
//     leader's token barrier, which counts its own bytes + this report), "my expanded weights are
//     in tensor memory" (each dequant warp arrives on the LEADER's barrier, count 8), "my epilogue
//     drained the accumulator" (count 8 on the leader).
//   * leader -> both: one tcgen05.commit with an arrival mask per barrier releases the token stage,
//     the A buffer and the accumulator in both CTAs. The MMA thread issues 8 MMAs + 2 commits and
//     probes two barriers per K stage: a thread issues one tcgen05 instruction per ~65 cycles, so
//     every instruction saved there counted (4 commits and 3 waits per stage ran 10 % slower).
// The ragged last token tile of an expert runs with a narrower MMA N (its rows rounded up to 32).
// Both CTAs run every role except MMA issue (leader only); the peer's idle MMA warp is the relay.
// Every wait is bounded; both CTAs meet at a cluster barrier before tensor memory is released.
#include <cuda_bf16.h>

#include <cstdio>
#include <cstdlib>

#include "cluster.cuh"
#include "common.cuh"
#include "kernels.h"
#include "tile_sched.cuh"

namespace xmoe {

#ifdef XMOE_TRACE
// Debug build only: per-cluster cycle totals of where the leader's MMA thread waits.
__device__ long long g_ff2p_trace[148 * 8];
#define XMOE_T0() const long long t0__ = clock64()
#define XMOE_TACC(var) var += clock64() - t0__
#else
#define XMOE_T0() do {} while (0)
#define XMOE_TACC(var) do {} while (0)
#endif

namespace {

constexpr int kBlockM = 128;             // weight rows per CTA
constexpr int kTokHalf = 128;            // token rows staged per CTA
constexpr int kTokTile = 256;            // token rows per pair tile = MMA N
constexpr int kStageK = 128;             // one int4 group
constexpr int kRawBytes = kBlockM * kStageK / 2;
constexpr int kWStageBytes = kRawBytes + 512;
constexpr int kBStageBytes = kTokHalf * kStageK * 2;   // 32 KiB: two 128-byte-swizzle slabs
constexpr int kWStages = 4;  // a multiple of kDqGroups: every weight slot always meets the same group (parity waits)
constexpr int kBStages = 5;
constexpr int kACols = kStageK / 2;      // 64
constexpr int kARing = 4;
constexpr int kDqGroups = 4;
constexpr int kAccBase = kARing * kACols;  // 256
static_assert(kWStages % kDqGroups == 0 && kARing % kDqGroups == 0, "ring slots must stay with one dequant group");
constexpr int kTmemCols = 512;
// warps: 0 weight producer, 1 MMA issuer / relay, 2-5 and 7-10 epilogue (two sets of four, one warp per tensor-memory
// lane quadrant in each set; the sets take alternate 32-token chunks of a tile), 6 token producer, 11-26 dequantisers
constexpr int kEpiSets = 2;
constexpr int kFirstDqWarp = 7 + 4 * (kEpiSets - 1);
constexpr int kThreads = 32 * (kFirstDqWarp + 4 * kDqGroups);  // 864
constexpr int kTailBytes = 5120;  // barriers + tile prefix
constexpr size_t kSmemBytes = 1024 + (size_t)kBStages * kBStageBytes + (size_t)kWStages * kWStageBytes + kTailBytes;
static_assert(kSmemBytes <= 232448, "shared memory");
static_assert(kAccBase + kTokTile <= kTmemCols, "TMEM budget");

// MMA N of a token tile: its valid rows rounded up to 32, at most 256 (both CTAs derive it from the tile).
__device__ __forceinline__ int tile_n_eff(const TileInfo& t) {
    const int n_valid = t.count - t.nt_idx * kTokTile;
    return n_valid >= kTokTile ? kTokTile : ((n_valid + 31) & ~31);
}

__device__ __forceinline__ __nv_bfloat162 bf162_from_bits(uint32_t bits) {
    __nv_bfloat162 v;
    memcpy(&v, &bits, 4);
    return v;
}
__device__ __forceinline__ uint32_t bits_from_bf162(__nv_bfloat162 v) {
    uint32_t bits;
    memcpy(&bits, &v, 4);
    return bits;
}
__device__ __forceinline__ uint4 lds_u128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
// (x & 0x000f000f) | 0x43004300 as ONE logic instruction: the two bf16 values 128 + nibble. Left
// to the compiler, the and and the or came out as two instructions per pair.
__device__ __forceinline__ uint32_t nib_pair_to_bf16_bits(uint32_t x) {
    uint32_t bits;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(bits) : "r"(x), "r"(0x000f000fu), "r"(0x43004300u));
    return bits;
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
// One 32-bit word of the prepared layout (8 weights: nibble j = K 2j, nibble 4 + j = K 2j + 1) -> four bf16x2
// registers bf16((u4 - 8) * scale), K ascending.
__device__ __forceinline__ void expand_word(uint32_t w, uint32_t* o, __nv_bfloat162 bias, __nv_bfloat162 s2) {
    o[0] = bits_from_bf162(__hmul2(__hsub2(bf162_from_bits(nib_pair_to_bf16_bits(w)), bias), s2));
    o[1] = bits_from_bf162(__hmul2(__hsub2(bf162_from_bits(nib_pair_to_bf16_bits(w >> 4)), bias), s2));
    o[2] = bits_from_bf162(__hmul2(__hsub2(bf162_from_bits(nib_pair_to_bf16_bits(w >> 8)), bias), s2));
    o[3] = bits_from_bf162(__hmul2(__hsub2(bf162_from_bits(nib_pair_to_bf16_bits(w >> 12)), bias), s2));
}

// 2-SM MMA: D (256 x N, 128 rows in each CTA's tensor memory) (+)= A (each CTA's tensor memory)
// * B (N/2 rows in each CTA's shared memory at the same offset).
__device__ __forceinline__ void mma_bf16_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], db, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHiSw128)
        : "memory");
}

__global__ __launch_bounds__(kThreads, 1) void ff2_w4a16_pair_kernel(const __grid_constant__ Ff2Args a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* b_base = smem;
    uint8_t* w_base = smem + (size_t)kBStages * kBStageBytes;
    uint8_t* tail = w_base + (size_t)kWStages * kWStageBytes;
    uint64_t* w_full = reinterpret_cast<uint64_t*>(tail);  // [16] local: raw weights + scales landed
    uint64_t* w_empty = w_full + 16;                       // [16] local: dequant group done with them
    uint64_t* b_full = w_empty + 16;                       // [8]  my token half landed (leader: and the peer's)
    uint64_t* b_empty = b_full + 8;                         // [8]  each CTA: MMAs reading the stage retired
    uint64_t* adq_full = b_empty + 8;                      // [8]  leader: both CTAs' expanded weights are in TMEM
    uint64_t* adq_empty = adq_full + 8;                    // [8]  each CTA: MMAs reading the A buffer retired
    uint64_t* acc_full = adq_empty + 8;                    // [1]  each CTA
    uint64_t* acc_empty = acc_full + 1;                    // [1]  leader: both epilogues drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    int* prefix = reinterpret_cast<int*>(tail + 640);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int cluster_id = blockIdx.x >> 1;
    const int n_clusters = gridDim.x >> 1;
    const int mt_tiles = (a.H + kBlockM - 1) / kBlockM;
    const int h_pairs = (mt_tiles + 1) / 2;
    const int k_stages = (a.I + kStageK - 1) / kStageK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kWStages; ++s) {
            mbar_init(&w_full[s], 1);
            mbar_init(&w_empty[s], 4);
        }
        for (int s = 0; s < kBStages; ++s) {
            // leader: its own TMA bytes + the peer's report that its half has landed
            mbar_init(&b_full[s], leader ? 2 : 1);
            mbar_init(&b_empty[s], 1);
        }
        for (int s = 0; s < kARing; ++s) {
            mbar_init(&adq_full[s], 8);
            mbar_init(&adq_empty[s], 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 2 * 4 * kEpiSets);
        *abort_flag = 0u;
        mbar_fence_init();
        prefetch_tmap(&a.tm_w);
        prefetch_tmap(&a.tm_y);
        prefetch_tmap(&a.tm_y_small);
        prefetch_tmap(&a.tm_y_mid);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, kTmemCols);
        tmem_relinquish_pair();
    }
    if (warp == 2) tile_prefix_build(prefix, a.counts, a.E_tot, h_pairs, kTokTile);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers are initialised before anyone arrives on them remotely
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int total_tiles = prefix[a.E_tot];

    if (warp == 0) {
        // ------------------------------ weight producer (my 128 rows) --------------
        if (lane == 0) {
            const uint16_t* scales = reinterpret_cast<const uint16_t*>(a.w2_scale);
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (int item = cluster_id; item < total_tiles && ok; item += n_clusters) {
                const TileInfo t = tile_decode(item, prefix, a.counts, a.offsets, a.E_tot, kTokTile);
                const int h0 = (t.wt * 2 + (int)rank) * kBlockM;
                const int w_row = t.e * a.H + h0;
                const int rows_here = max(0, min(kBlockM, a.H - h0));
                const uint32_t scale_bytes = (uint32_t)rows_here * 2u;
                for (int ks = 0; ks < k_stages; ++ks) {
                    if (!mbar_wait(&w_empty[s], ph ^ 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_MMA)) {
                        ok = false;
                        break;
                    }
                    uint8_t* st = w_base + (size_t)s * kWStageBytes;
                    mbar_expect_tx(&w_full[s], kRawBytes + scale_bytes);
                    tma_load_2d(st, &a.tm_w, ks * (kStageK / 2), w_row, &w_full[s]);
                    if (scale_bytes)
                        tma_load_1d(st + kRawBytes, scales + ((size_t)t.e * a.groups + ks) * a.H + h0, scale_bytes,
                                    &w_full[s]);
                    if (++s == (uint32_t)kWStages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 6) {
        // ------------------------------ token producer (my 128 token rows) --------
        if (lane == 0) {
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (int item = cluster_id; item < total_tiles && ok; item += n_clusters) {
                const TileInfo t = tile_decode(item, prefix, a.counts, a.offsets, a.E_tot, kTokTile);
                // each CTA stages half of the tile's MMA N: the smallest of the 32-, 64- and 128-row boxes that holds it
                const int half = tile_n_eff(t) >> 1;
                const int row = t.row0 + (int)rank * half;
                const CUtensorMap* tm = half <= 32 ? &a.tm_y_small : (half <= 64 ? &a.tm_y_mid : &a.tm_y);
                const uint32_t stage_bytes = (half <= 32 ? 32u : (half <= 64 ? 64u : 128u)) * 256u;  // two slabs of K 64
                for (int ks = 0; ks < k_stages; ++ks) {
                    if (!mbar_wait(&b_empty[s], ph ^ 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_MMA)) {
                        ok = false;
                        break;
                    }
                    uint8_t* b = b_base + (size_t)s * kBStageBytes;
                    mbar_expect_tx(&b_full[s], stage_bytes);
                    tma_load_3d(b, tm, 0, row, ks * (kStageK / 64), &b_full[s]);  // zero-filled beyond I
                    if (++s == (uint32_t)kBStages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            // ------------------------------ MMA issuer (leader CTA) -----------------
            const uint32_t b_lo0 = umma_desc_lo_sw128(smem_u32(b_base));
            uint32_t tile_n = 0, s = 0, ph = 0, d = 0, dph = 0;
            bool ok = true;
#ifdef XMOE_TRACE
            long long tw_b = 0, tw_bp = 0, tw_adq = 0, tw_acc = 0, t_issue = 0;
            const long long t_start = clock64();
#endif
            for (int item = cluster_id; item < total_tiles && ok; item += n_clusters, ++tile_n) {
                // the ragged last token tile of an expert runs with a narrower N (cost ~ N, floor at the
                // issue rate): each CTA then stages N/2 of its rows instead of 128. Decoded before the wait for the
                // accumulator, i.e. while the epilogue of the previous tile runs.
                int n_eff;
                {
                    XMOE_T0();
                    n_eff = tile_n_eff(tile_decode(item, prefix, a.counts, a.offsets, a.E_tot, kTokTile));
                    XMOE_TACC(tw_bp);
                }
                {
                    XMOE_T0();
                    if (!mbar_wait_cluster(acc_empty, (tile_n & 1u) ^ 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_EPI)) break;
                    XMOE_TACC(tw_acc);
                }
                tc_fence_after();
                const uint32_t acc = tmem_base + kAccBase;
                const uint32_t idesc = umma_idesc_bf16(2 * kBlockM, (uint32_t)n_eff);
                // distance between the two K 64 slabs of a stage, in 16-byte units: the rows of the box the producers used
                const uint32_t slab16 = (n_eff <= 64 ? 32u : (n_eff <= 128 ? 64u : 128u)) * 8u;
                for (int ks = 0; ks < k_stages; ++ks) {
                    {
                        XMOE_T0();
                        if (!mbar_wait(&b_full[s], ph, abort_flag, a.status, XMOE_DEV_TIMEOUT_TMA)) { ok = false; break; }
                        XMOE_TACC(tw_b);
                    }
                    {
                        XMOE_T0();
                        if (!mbar_wait_cluster(&adq_full[d], dph, abort_flag, a.status, XMOE_DEV_TIMEOUT_DQ)) { ok = false; break; }
                        XMOE_TACC(tw_adq);
                    }
                    XMOE_T0();
                    tc_fence_after();
                    const uint32_t a_tmem = tmem_base + d * kACols;
                    const uint32_t b_lo = b_lo0 + s * (uint32_t)(kBStageBytes >> 4);
#pragma unroll
                    for (int kk = 0; kk < kStageK / 16; ++kk)
                        mma_bf16_ts_pair(acc, a_tmem + kk * 8, b_lo + (kk >> 2) * slab16 + (kk & 3) * 2, idesc,
                                         (ks | kk) ? 1u : 0u);
                    // release the token stage and the A buffer in both CTAs
                    tc_commit_pair_mask(smem_u32(&b_empty[s]), 3);
                    tc_commit_pair_mask(smem_u32(&adq_empty[d]), 3);
                    if (++s == (uint32_t)kBStages) { s = 0; ph ^= 1u; }
                    if (++d == (uint32_t)kARing) { d = 0; dph ^= 1u; }
                    XMOE_TACC(t_issue);
                }
                if (ok) tc_commit_pair_mask(smem_u32(acc_full), 3);
            }
#ifdef XMOE_TRACE
            if (cluster_id < 148) {
                long long* o = g_ff2p_trace + cluster_id * 8;
                o[0] = tw_b; o[1] = tw_bp; o[2] = tw_adq; o[3] = tw_acc; o[4] = t_issue; o[5] = clock64() - t_start;
                o[6] = tile_n;
            }
#endif
        } else if (lane == 0) {
            // ------------------------------ relay (peer CTA) -------------------------
            // tells the leader when this CTA's half of a token stage has landed
            const uint32_t leader_b_full = map_to_cta(smem_u32(&b_full[0]), 0);
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (int item = cluster_id; item < total_tiles && ok; item += n_clusters) {
                for (int ks = 0; ks < k_stages; ++ks) {
                    if (!mbar_wait(&b_full[s], ph, abort_flag, a.status, XMOE_DEV_TIMEOUT_TMA)) {
                        ok = false;
                        break;
                    }
                    mbar_arrive_cluster(leader_b_full + s * 8u);
                    if (++s == (uint32_t)kBStages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp < kFirstDqWarp) {
        // ------------------------------ epilogue (my 128 features x 256 tokens) -----
        // tcgen05.ld gives a thread one feature (lane) of 32 tokens (registers), so store j of a warp writes 32
        // consecutive bf16 (64 bytes, two whole sectors) of token j's output row: no transpose. A row's home is this
        // GPU's row buffer or (expert parallel) a peer's return buffer; the addresses are fetched once per chunk by
        // the lane of the token's number and handed round by shuffle. 64 contiguous bytes per instruction also suit
        // peer memory over NVLink (lanes each storing 16-byte pieces of different rows did not: 0.83 against
        // 0.69 ms with 7/8 of the rows remote; staging whole 256-byte segments through shared memory was slower
        // than this at 2 and at 8 GPUs). Two sets of four warps take the 32-token chunks of a tile alternately (a
        // warp reaches the lane quadrant warp % 4 of tensor memory): the accumulator is single, so the MMAs of the
        // next tile wait for the whole drain.
        const int q = warp & 3;
        const int set = warp < 6 ? 0 : 1;
        uint32_t tile_n = 0;
        uint16_t* out = reinterpret_cast<uint16_t*>(a.out);
        const uint32_t leader_acc_empty = map_to_cta(smem_u32(acc_empty), 0);
        for (int item = cluster_id; item < total_tiles; item += n_clusters, ++tile_n) {
            const TileInfo t = tile_decode(item, prefix, a.counts, a.offsets, a.E_tot, kTokTile);
            if (!mbar_wait_cluster(acc_full, tile_n & 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_ACC)) break;
            tc_fence_after();
            const int h = (t.wt * 2 + (int)rank) * kBlockM + q * 32 + lane;  // this lane's feature
            const bool h_ok = h < a.H;
            const int n_valid = min(kTokTile, t.count - t.nt_idx * kTokTile);
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + kAccBase;
#ifdef XMOE_TRACE
            const long long te0 = clock64();
#endif
            // Halves of 16 tokens in two register sets: while one half is stored the next one is already on its way
            // from tensor memory, and the accumulator goes back to the MMA thread as soon as the LAST half has been
            // read, before it is stored.
            const int c_first = set * 32;
            bool released = false;
            if (c_first < n_valid) {
                uint32_t va[16], vb[16];
                tmem_ld16(lane_addr + c_first, va);
                for (int c0 = c_first; c0 < n_valid; c0 += 32 * kEpiSets) {
                    const int prow = t.row0 + c0 + lane;
                    unsigned long long my_row = 0ull;
                    if (c0 + lane < n_valid)
                        my_row = a.row_dst ? a.row_dst[prow] : (unsigned long long)(uintptr_t)(out + (size_t)prow * a.H);
                    tmem_ld_wait();                          // va: tokens c0 .. c0 + 15
                    tmem_ld16(lane_addr + c0 + 16, vb);      // tokens c0 + 16 .. c0 + 31, in flight during the stores of va
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const unsigned long long row = __shfl_sync(0xffffffffu, my_row, j);
                        if (row && h_ok)
                            reinterpret_cast<uint16_t*>((uintptr_t)row)[h] = (uint16_t)f32_to_bf16_bits(__uint_as_float(va[j]));
                    }
                    tmem_ld_wait();                          // vb
                    const int c_next = c0 + 32 * kEpiSets;
                    if (c_next < n_valid) {
                        tmem_ld16(lane_addr + c_next, va);   // next chunk's first half, in flight during the stores of vb
                    } else {
                        // every column this warp reads has been read
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(leader_acc_empty);
                        released = true;
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const unsigned long long row = __shfl_sync(0xffffffffu, my_row, 16 + j);
                        if (row && h_ok)
                            reinterpret_cast<uint16_t*>((uintptr_t)row)[h] = (uint16_t)f32_to_bf16_bits(__uint_as_float(vb[j]));
                    }
                }
            }
#ifdef XMOE_TRACE
            if (warp == 2 && lane == 0 && cluster_id < 148 && leader) g_ff2p_trace[cluster_id * 8 + 7] += clock64() - te0;
#endif
            if (!released) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(leader_acc_empty);
            }
        }
    } else {
        // ------------------------------ dequantiser (my 128 rows -> my tensor memory) --
        const int quadrant = warp & 3;
        const int group = (warp - kFirstDqWarp) >> 2;
        const int row = quadrant * 32 + lane;
        const uint32_t swz = (uint32_t)(row >> 1) & 3u;  // 64-byte TMA swizzle: 16-byte chunk ^= (row / 2) % 4
        const __nv_bfloat162 bias = bf162_from_bits(0x43084308u);  // 136.0 twice
        const uint32_t leader_adq_full = map_to_cta(smem_u32(&adq_full[0]), 0);
        // the K stages of all tiles of this cluster are numbered through; this group takes
        // it = group, group + kDqGroups, ... without walking the stages of the other groups
        const int my_tiles = cluster_id < total_tiles ? (total_tiles - 1 - cluster_id) / n_clusters + 1 : 0;
        const uint32_t total_it = (uint32_t)my_tiles * (uint32_t)k_stages;
        const uint32_t w_base_u32 = smem_u32(w_base);
        {
            for (uint32_t it = (uint32_t)group; it < total_it; it += kDqGroups) {
                const int s = it % kWStages;
                const uint32_t ph = (it / kWStages) & 1u;
                const int d = it % kARing;
                const uint32_t dph = (it / kARing) & 1u;
                if (!mbar_wait(&w_full[s], ph, abort_flag, a.status, XMOE_DEV_TIMEOUT_TMA) ||
                    !mbar_wait_cluster(&adq_empty[d], dph ^ 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_DQ))
                    break;
                tc_fence_after();
                const uint32_t st = w_base_u32 + (uint32_t)s * kWStageBytes;
                const uint32_t sraw = lds_u16(st + kRawBytes + row * 2);
                const __nv_bfloat162 s2 = bf162_from_bits(__byte_perm(sraw, sraw, 0x1010));
                const uint32_t a_lane = tmem_base + ((uint32_t)(quadrant * 32) << 16) + d * kACols;
                // 16 bytes (32 weights) at a time: four words -> sixteen bf16x2 registers -> one 16-column store
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint4 r4 = lds_u128(st + row * 64 + (((uint32_t)q ^ swz) * 16));
                    uint32_t o[16];
                    expand_word(r4.x, o, bias, s2);
                    expand_word(r4.y, o + 4, bias, s2);
                    expand_word(r4.z, o + 8, bias, s2);
                    expand_word(r4.w, o + 12, bias, s2);
                    tmem_st16(a_lane + q * 16, o);
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive_cluster(leader_adq_full + d * 8u);  // the leader issues the MMAs of both CTAs
                    mbar_arrive(&w_empty[s]);
                }
            }
        }
    }

    // both CTAs finish every remote access before either releases tensor memory or exits
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    cluster_sync_all();
    if (warp == 1) tmem_dealloc_pair(tmem_base, kTmemCols);
}

}  // namespace

#ifdef XMOE_TRACE
extern "C" int xmoe_ff2_pair_trace_dump(long long* host_out) {
    return (int)cudaMemcpyFromSymbol(host_out, g_ff2p_trace, sizeof(g_ff2p_trace));
}
#endif

int launch_ff2_pair(const Ff2Args& a, cudaStream_t stream) {
    static bool attr_set_dev[kMaxDevices] = {};
    const int dev = device_slot();
    if (dev < 0) return XMOE_ERR_CUDA;
    bool& attr_set = attr_set_dev[dev];
    if (!attr_set) {
        if (cudaFuncSetAttribute(ff2_w4a16_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
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
        if (cudaOccupancyMaxActiveClusters(&n, ff2_w4a16_pair_kernel, &cfg) != cudaSuccess || n <= 0) n = a.num_sms / 2;
        resident_clusters = n < a.num_sms / 2 ? n : a.num_sms / 2;
        if (getenv("XMOE_DEBUG")) fprintf(stderr, "xmoe: ff2 pair kernel: %d resident clusters of 2 CTAs (occupancy query %d, %d SMs)\n", resident_clusters, n, a.num_sms);
    }
    cfg.gridDim = dim3((unsigned)(2 * resident_clusters), 1, 1);
    return cudaLaunchKernelEx(&cfg, ff2_w4a16_pair_kernel, a) == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

}  // namespace xmoe
