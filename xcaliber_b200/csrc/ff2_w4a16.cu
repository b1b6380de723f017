// FF2: grouped W4A16 down projection. int4 group-128 weights are expanded to bf16 on the
// way into TENSOR MEMORY (the MMA's A operand), activations are the bf16 FF1 output staged
// by TMA; accumulation is bf16 x bf16 -> fp32 on tcgen05.
//
// Weight contract: symmetric int4, group 128 along K, w = (u4 - 8) * scale[k/128] -- the
// GPTQ / compressed-tensors contract of the reference's INT4 lane
// (xFused-XXXX-Kernels/xMoE/xW4A16/sm75/xR64/xR64ABSRepack.cu:3-24, xR64ABS.cuh:30-34,
// vllm/xcaliber_int4_vllm/method.py:188-203). The "expand 4-bit weights with a few logic
// ops, then use the 16-bit tensor path" idea is the one the reference sketches in
// xFused-NVFP4-Kernels/ptx.cuh:1-83; here the expansion is the integer flavour:
// (nibble | 0x4300) is the bf16 value 128 + nibble, minus 136 gives nibble - 8 exactly, one
// bf16x2 multiply applies the group scale (a single rounding, i.e. bf16((u4 - 8) * s)).
//
// Structure (128 output features = MMA M, NT packed token rows = MMA N):
//   warp 0      weight producer: TMA of the raw int4 tile (128 rows x K/2 bytes, swizzled so
//               that one thread per row reads without bank conflicts) + its bf16 group scales
//               into a DEEP ring (the weights come from HBM)
//   warp 6      token producer: TMA of the bf16 activation tile (NT x K, 128-byte swizzle) into a
//               SHORT ring (the activations come from L2)
//   warps 7..   dequantise (groups of 4 warps, stages round-robin): thread = weight row; the
//               bf16 pairs go straight to tensor memory with tcgen05.st (lane = row, column =
//               K pair). Expanded weights never touch shared memory (a bf16 tile written to
//               shared memory costs 10 B of shared-memory traffic per weight byte).
//   warp 1      tcgen05.mma kind::f16 with A from tensor memory, B from shared memory. Token
//               tiles of 32 / 64 rows add three more issuing warps (7-9; the dequant warps then
//               start at 10) that take the K stages round-robin into separate accumulators,
//               which the epilogue adds in a fixed order: one thread issues at most one MMA per
//               ~70 cycles, far below what the tensor pipe takes for N = 32.
//   warps 2-5   epilogue: tcgen05.ld (lane = output feature, register = token), bf16 stores of 64
//               contiguous bytes per warp instruction to [packed row, H]
// All mbarrier waits are bounded (see common.cuh).
#include <cuda_bf16.h>

#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "tile_sched.cuh"

namespace xmoe {

#ifdef XMOE_TRACE
// Debug build only: per-CTA cycle totals of where each role waits.
__device__ long long g_ff2_trace[148 * 16];
#define XMOE_T0() const long long t0__ = clock64()
#define XMOE_TACC(var) var += clock64() - t0__
#define XMOE_T1() const long long t1__ = clock64()
#define XMOE_TACC1(var) var += clock64() - t1__
#define XMOE_TDUMP(slot, var) do { if (blockIdx.x < 148) g_ff2_trace[blockIdx.x * 16 + (slot)] = (var); } while (0)
#else
#define XMOE_T0() do {} while (0)
#define XMOE_TACC(var) do {} while (0)
#define XMOE_T1() do {} while (0)
#define XMOE_TACC1(var) do {} while (0)
#define XMOE_TDUMP(slot, var) do {} while (0)
#endif

namespace {

constexpr int kBlockM = 128;
constexpr int kMaxExperts = 1024 + 8;
constexpr int kTmemCols = 512;
constexpr int kTailBytes = 5120;  // barriers + tile prefix
constexpr int kFirstDqWarp = 7;

// NT <= 128: one K stage = one int4 group (K 128). NT = 128 has two accumulators (the epilogue
// overlaps the next tile) or, as TWO_ISSUERS, one accumulator for each of two issuing threads; NT = 32 / 64
// spend the tensor-memory columns on one accumulator per issuing thread (four). NT = 256 (long-K prefill): a single issuing thread sustains one K=16
// MMA per ~70 cycles at best, so only N = 256 (128 cycles of tensor pipe) runs the bf16 pipe at
// full rate; the 256-column accumulator is then single and the stages are K 64.
template <int NT, bool TWO_ISSUERS = false>
struct Ff2Cfg {
    static_assert(!TWO_ISSUERS || NT <= 128, "the two-issuer variant exists for token tiles of 32, 64 and 128");
    static constexpr int kStageK = NT >= 256 ? 64 : 128;
    static constexpr int kRawBytes = kBlockM * kStageK / 2;   // int4 tile: 128 rows x kStageK/2 bytes
    // Small token tiles are HBM-bound: their weight stage spans two K units, so that every row
    // contributes a whole 128-byte line per TMA request (64-byte pieces ran HBM at half rate).
    static constexpr int kWUnits = NT <= 64 ? 2 : 1;
    static constexpr int kWRowBytes = kWUnits * kStageK / 2;  // bytes of one weight row in a stage
    static constexpr int kWRawBytes = kWUnits * kRawBytes;
    static constexpr int kWStageBytes = kWRawBytes + 512 * kWUnits;  // + 128 bf16 scales per unit, padded
    static constexpr int kACols = kStageK / 2;                // TMEM columns of one expanded stage
    static constexpr int kSlabs = kStageK / 64;               // 128-byte-swizzle slabs of the token tile
    // a token stage spans the same K units as a weight stage (small tiles: two, fetched by ONE copy through a
    // 3-D view of the activations): the copy engine takes ~100-200 cycles per request whatever its size, and with
    // two slab copies per K unit the token producer alone set the pace of the decode kernel
    static constexpr int kBStageBytes = NT * kStageK * 2 * kWUnits;
#ifndef XMOE_FF2_WS32
#define XMOE_FF2_WS32 8
#endif
#ifndef XMOE_FF2_BS32
#define XMOE_FF2_BS32 4
#endif
#ifndef XMOE_FF2_WS64
#define XMOE_FF2_WS64 8
#endif
#ifndef XMOE_FF2_BS64
#define XMOE_FF2_BS64 2
#endif
#ifndef XMOE_FF2_SPLIT
#define XMOE_FF2_SPLIT 1
#endif


    static constexpr int kWStages = NT == 128 ? (TWO_ISSUERS ? 8 : 12) : (NT == 64 ? XMOE_FF2_WS64 : (NT == 32 ? XMOE_FF2_WS32 : 16));  // weight ring (HBM latency)
    static constexpr int kBStages = NT >= 256 ? 4 : (NT >= 128 ? (TWO_ISSUERS ? 4 : 3) : (NT == 32 ? XMOE_FF2_BS32 : XMOE_FF2_BS64));  // token ring (L2 latency)
    static constexpr int kIssuers = TWO_ISSUERS ? 2 : (NT <= 64 ? 4 : 1);         // MMA-issuing threads (K stages round-robin)
    static constexpr int kARing = NT >= 256 ? 8 : 4;          // expanded-weight buffers in tensor memory
    // Small token tiles hand a buffer over in two halves (K 64 each, own barriers): the issuer starts on the
    // first half while the second is still being expanded, and the dequant group gets the first half back
    // before it has finished the second, so expansion and MMA issue of one group overlap instead of taking
    // turns on the buffer (tensor memory has no room for a second whole buffer per group).
    static constexpr int kSplit = NT <= 64 ? XMOE_FF2_SPLIT : 1;
    static constexpr int kDqGroups = 4;                       // independent dequant groups of 4 warps
    // Ring ownership. The waits are parity waits, and a parity only tells a phase from its
    // neighbours: a role may wait on a slot only if it took part in that slot's previous phase
    // (or something else orders it after that phase), otherwise a role that runs ahead reads
    // "complete" from the phase before last. So every slot of a ring always belongs to the same
    // role instance. All roles number the K stages of a CTA's tiles through with one counter in
    // which every tile takes k_walk = K stages rounded up to kWUnits slots: with two K units per
    // weight stage and an odd stage count the last slot of a tile is a PHANTOM stage, walked by
    // every role with its barrier hand-offs but without loads, expansion or MMAs. Then stage
    // number = 2 * weight stage + unit, group = stage % 4 owns tensor-memory slot stage % kARing
    // and always meets the same weight slots (kARing and the weight ring are multiples of
    // kDqGroups). The token ring and kARing are multiples of kIssuers, and an issuing thread takes the
    // units whose CTA-wide number is its own index modulo kIssuers (not the position inside the tile), so
    // that it, too, always meets the same token and tensor-memory slots, whatever the tile lengths.
    // two accumulator sets where tensor memory has room (NT 128: 2 x 128 columns; NT 32: 2 x 4 issuers x 32): the
    // epilogue of one tile (or tile segment) overlaps the MMAs of the next
    static constexpr int kAccStages = NT <= 64 ? 256 / (kIssuers * NT) : ((NT == 128 && !TWO_ISSUERS) ? 2 : 1);
    static constexpr int kFirstDq = kFirstDqWarp + (kIssuers - 1);
    static constexpr int kThreads = 32 * (kFirstDq + 4 * kDqGroups);
    static constexpr int kAccBase = kARing * kACols;          // accumulators follow the A ring
    static_assert(kAccBase + kAccStages * kIssuers * NT <= kTmemCols, "TMEM budget");
    static_assert(kWStages <= 16 && kBStages <= 16 && kARing * kSplit <= 8, "barrier arrays");
    static_assert(kSplit == 1 || (kStageK / 32) % kSplit == 0, "halves are whole 16-column stores");
    static_assert(kThreads <= 1024, "block size");
    static_assert(kARing % kDqGroups == 0 &&
                      (kIssuers == 1 || (kARing % kIssuers == 0 && (kBStages * kWUnits) % kIssuers == 0)),
                  "ring ownership");
    static_assert((kWStages * kWUnits) % kDqGroups == 0, "weight ring ownership");
    static constexpr size_t kSmemBytes =
        1024 + (size_t)kBStages * kBStageBytes + (size_t)kWStages * kWStageBytes + kTailBytes;
    static_assert(kSmemBytes <= 232448, "shared memory");
};

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
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// polls (~100 ns each) a finishing CTA spends on one helper's flag before it gives up: ~0.2 s
constexpr uint32_t kPartialSpinLimit = 1u << 21;
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
// One 32-bit word of the prepared layout (8 weights: nibble j = K 2j, nibble 4 + j = K 2j + 1) -> four bf16x2
// registers bf16((u4 - 8) * scale), K ascending: per pair one logic op, one subtract, one multiply, and a shift
// for three of the four.
__device__ __forceinline__ void expand_word(uint32_t w, uint32_t* o, __nv_bfloat162 bias, __nv_bfloat162 s2) {
    o[0] = bits_from_bf162(__hmul2(__hsub2(bf162_from_bits(nib_pair_to_bf16_bits(w)), bias), s2));
    o[1] = bits_from_bf162(__hmul2(__hsub2(bf162_from_bits(nib_pair_to_bf16_bits(w >> 4)), bias), s2));
    o[2] = bits_from_bf162(__hmul2(__hsub2(bf162_from_bits(nib_pair_to_bf16_bits(w >> 8)), bias), s2));
    o[3] = bits_from_bf162(__hmul2(__hsub2(bf162_from_bits(nib_pair_to_bf16_bits(w >> 12)), bias), s2));
}

template <int NT, bool KSPLIT, bool TWO_ISSUERS>
__global__ __launch_bounds__(Ff2Cfg<NT, TWO_ISSUERS>::kThreads, 1) void ff2_w4a16_kernel(const __grid_constant__ Ff2Args a) {
    static_assert(!KSPLIT || NT <= 64, "tiles are cut along K only for small token tiles");
    using Cfg = Ff2Cfg<NT, TWO_ISSUERS>;
    constexpr int kARing = Cfg::kARing, kDqGroups = Cfg::kDqGroups, kAccBase = Cfg::kAccBase;
    constexpr int kStageK = Cfg::kStageK, kACols = Cfg::kACols;
    constexpr int kAccStages = Cfg::kAccStages, kWStages = Cfg::kWStages, kBStages = Cfg::kBStages;
    constexpr int kIssuers = Cfg::kIssuers;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* b_base = smem;                                          // token ring
    uint8_t* w_base = smem + (size_t)kBStages * Cfg::kBStageBytes;   // weight ring
    uint8_t* tail = w_base + (size_t)kWStages * Cfg::kWStageBytes;
    uint64_t* w_full = reinterpret_cast<uint64_t*>(tail);  // [16] raw weights + scales landed
    uint64_t* w_empty = w_full + 16;                       // [16] the 4 warps of a dequant group are done with them
    uint64_t* b_full = w_empty + 16;                       // [16] token tile landed
    uint64_t* b_empty = b_full + 16;                       // [16] MMAs reading it retired
    uint64_t* adq_full = b_empty + 16;                     // [8]  expanded weights are in tensor memory
    uint64_t* adq_empty = adq_full + 8;                    // [8]  MMAs reading them retired
    uint64_t* acc_full = adq_empty + 8;                    // [4]
    uint64_t* acc_empty = acc_full + 4;                    // [4]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 4);
    static_assert(kAccStages <= 4, "accumulator barrier arrays");
    volatile uint32_t* abort_flag = tmem_slot + 1;
    int* prefix = reinterpret_cast<int*>(tail + 768);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int mt_tiles = (a.H + kBlockM - 1) / kBlockM;
    const int k_stages = (a.I + kStageK - 1) / kStageK;
    // slots per tile in the CTA-wide stage numbering (see "Ring ownership"): slots >= k_stages are phantoms
    const int k_walk = (k_stages + Cfg::kWUnits - 1) / Cfg::kWUnits * Cfg::kWUnits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kWStages; ++s) {
            mbar_init(&w_full[s], 1);
            mbar_init(&w_empty[s], 4 * Cfg::kWUnits);
        }
        for (int s = 0; s < kBStages; ++s) {
            mbar_init(&b_full[s], 1);
            mbar_init(&b_empty[s], Cfg::kWUnits);  // one commit per K unit of the stage (each from the unit's issuer)
        }
        for (int s = 0; s < kARing * Cfg::kSplit; ++s) {  // index: buffer * kSplit + half
            mbar_init(&adq_full[s], 4);
            mbar_init(&adq_empty[s], 1);
        }
        for (int s = 0; s < kAccStages; ++s) {
            mbar_init(&acc_full[s], kIssuers);
            mbar_init(&acc_empty[s], 4);
        }
        *abort_flag = 0u;
        mbar_fence_init();
        prefetch_tmap(&a.tm_w);
        prefetch_tmap(&a.tm_y);
        if (NT <= 64 && a.scale2d) prefetch_tmap(&a.tm_s);
        if (NT <= 64) {
            prefetch_tmap(&a.tm_y_small);
            prefetch_tmap(&a.tm_y_mid);
        }
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
    // this CTA's share: whole tiles at a balanced stride, or (small token tiles with scratch for partial sums) an
    // equal run of K units that may cut tiles (tile_sched.cuh: KWalk)
    const int cta = (int)blockIdx.x;
    KWalk walk;
    {
        // cutting tiles costs one more segment (one more accumulator drain) per CTA: worth it only when whole tiles
        // would leave more than a tenth of the SM-rounds idle (256 tiles on 148 SMs: 13.5 %; 1173 tiles: 1 %) and a
        // tile is long enough (>= 32 K units) for the extra drain to be small against it, or there are fewer
        // tiles than SMs. KSPLIT is a separate instantiation: with the partial-sum code merely present, the
        // epilogue of short tiles (6 K units) ran a fifth slower
        const int grid = (int)gridDim.x;
        const int rounds = (total_tiles + grid - 1) / grid;
        const bool uneven = (k_walk >= 32 || total_tiles < grid) && total_tiles > 0 && total_tiles * 10 < grid * rounds * 9;
        walk.init(total_tiles, k_walk, grid, cta, KSPLIT && uneven);
    }

    if (warp == 0) {
        // ------------------------------ weight producer ---------------------------
        if (lane == 0) {
            const uint16_t* scales = reinterpret_cast<const uint16_t*>(a.w2_scale);
            uint32_t s = 0, ph = 0;
            bool ok = true;
            long long tw_prod = 0;
            (void)tw_prod;
            for (int si = 0; si < walk.n_seg && ok; ++si) {
                const KSegment sg = walk.seg(si, cta);
                const TileInfo t = tile_decode(sg.tile, prefix, a.counts, a.offsets, a.E_tot, NT);
                const int h0 = t.wt * kBlockM;
                const int w_row = t.e * a.H + h0;
                const int rows_here = min(kBlockM, a.H - h0);
                const uint32_t scale_bytes = (uint32_t)rows_here * 2u;  // H % 8 == 0 keeps this a multiple of 16
                for (int ks = sg.ks0; ks < sg.ks1 && ks < k_stages; ks += Cfg::kWUnits) {
                    {
                        XMOE_T0();
                        if (!mbar_wait(&w_empty[s], ph ^ 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_MMA)) {
                            ok = false;
                            break;
                        }
                        XMOE_TACC(tw_prod);
                    }
                    uint8_t* st = w_base + (size_t)s * Cfg::kWStageBytes;
                    if (Cfg::kWUnits == 2 && a.scale2d) {
                        // the scales of both K units in one request (a box of 2 groups x 128 features; beyond the
                        // tensor it is zero-filled, beyond the expert's groups it feeds a phantom unit): every
                        // request costs the copy engine about the same whatever its size
                        mbar_expect_tx(&w_full[s], Cfg::kWRawBytes + 512u);
                        tma_load_2d(st, &a.tm_w, ks * (kStageK / 2), w_row, &w_full[s]);
                        tma_load_2d(st + Cfg::kWRawBytes, &a.tm_s, h0, t.e * a.groups + ks, &w_full[s]);
                    } else {
                        const int units = min(Cfg::kWUnits, k_stages - ks);
                        mbar_expect_tx(&w_full[s], Cfg::kWRawBytes + (uint32_t)units * scale_bytes);
                        tma_load_2d(st, &a.tm_w, ks * (kStageK / 2), w_row, &w_full[s]);
                        for (int u = 0; u < units; ++u)
                            tma_load_1d(st + Cfg::kWRawBytes + u * 256,
                                        scales + ((size_t)t.e * a.groups + ((ks + u) * kStageK) / 128) * a.H + h0, scale_bytes,
                                        &w_full[s]);
                    }
                    if (++s == (uint32_t)kWStages) { s = 0; ph ^= 1u; }
                }
            }
            XMOE_TDUMP(0, tw_prod);
        }
    } else if (warp == 6) {
        // ------------------------------ token producer ----------------------------
        if (lane == 0) {
            uint32_t s = 0, ph = 0;
            bool ok = true;
            long long tw_bprod = 0;
            (void)tw_bprod;
            for (int si = 0; si < walk.n_seg && ok; ++si) {
                const KSegment sg = walk.seg(si, cta);
                const TileInfo t = tile_decode(sg.tile, prefix, a.counts, a.offsets, a.E_tot, NT);
                // Few tokens in the tile (decode): fetch only 8 or 16 rows. The token tile comes
                // from L2 at the same bytes per K as the weights do from HBM, and the L2 -> SM
                // path is shared by both.
                const CUtensorMap* tm = &a.tm_y;
                int box_rows = NT;
                if (NT <= 64) {
                    const int n_valid = t.count - t.nt_idx * NT;
                    if (n_valid <= 8) { tm = &a.tm_y_small; box_rows = 8; }
                    else if (n_valid <= 16) { tm = &a.tm_y_mid; box_rows = 16; }
                }
                const uint32_t slab_bytes = (uint32_t)box_rows * 128u;  // one slab: box_rows x 64 K
                for (int ks = sg.ks0; ks < sg.ks1; ks += Cfg::kWUnits) {
                    {
                        XMOE_T0();
                        if (!mbar_wait(&b_empty[s], ph ^ 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_MMA)) {
                            ok = false;
                            break;
                        }
                        XMOE_TACC(tw_bprod);
                    }
                    uint8_t* b = b_base + (size_t)s * Cfg::kBStageBytes;
                    if (Cfg::kWUnits > 1 && a.tok3d) {
                        // both K units in one request: four slabs, zero-filled beyond I
                        mbar_expect_tx(&b_full[s], slab_bytes * (uint32_t)(Cfg::kWUnits * Cfg::kSlabs));
                        tma_load_3d(b, tm, 0, t.row0, (ks * kStageK) >> 6, &b_full[s]);
                    } else {
                        const int units = min(Cfg::kWUnits, k_stages - ks);  // the phantom unit of an odd count is not fetched
                        mbar_expect_tx(&b_full[s], slab_bytes * (uint32_t)(units * Cfg::kSlabs));
                        for (int u = 0; u < units; ++u)
#pragma unroll
                            for (int slab = 0; slab < Cfg::kSlabs; ++slab)
                                tma_load_2d(b + (u * Cfg::kSlabs + slab) * slab_bytes, tm, (ks + u) * kStageK + slab * 64,
                                            t.row0, &b_full[s]);
                    }
                    if (++s == (uint32_t)kBStages) { s = 0; ph ^= 1u; }
                }
            }
            XMOE_TDUMP(1, tw_bprod);
        }
    } else if (warp == 1 || (kIssuers > 1 && warp >= kFirstDqWarp && warp < Cfg::kFirstDq)) {
        // ------------------------------ MMA issuer(s) ------------------------------
        // A thread can issue one MMA per ~70 cycles whatever its N, while an N = 32 MMA occupies
        // the tensor pipe for ~16: with small token tiles the issuing thread, not the pipe, would
        // bound the kernel. Small tiles therefore run kIssuers issuing threads that take the K
        // stages round-robin, each into its own accumulator; the epilogue adds the partial sums.
        if (lane == 0) {
            const int issuer = warp == 1 ? 0 : warp - kFirstDqWarp + 1;
            constexpr int kSlab16 = (NT * 128) >> 4;
            const uint32_t b_lo0 = umma_desc_lo_sw128(smem_u32(b_base));
            uint32_t tile_n = 0;
            bool ok = true;
            long long tw_full = 0, tw_adq = 0, tw_acc = 0, t_issue = 0;
            (void)tw_full; (void)tw_adq; (void)tw_acc; (void)t_issue;
            for (int si = 0; si < walk.n_seg && ok; ++si, ++tile_n) {
                const KSegment sg = walk.seg(si, cta);
                const uint32_t as = tile_n % kAccStages;
                const uint32_t aph = (tile_n / kAccStages) & 1u;
                // slab stride of this tile's token stages: the producer fetches 8 or 16 rows when the tile holds that few
                uint32_t slab16 = (uint32_t)kSlab16;
                uint32_t idesc = umma_idesc_bf16(kBlockM, NT);
                if (NT <= 64 || TWO_ISSUERS) {  // (decoded before the wait for the accumulator: the epilogue may still hold it)
                    const TileInfo t = tile_decode(sg.tile, prefix, a.counts, a.offsets, a.E_tot, NT);
                    const int n_valid = t.count - t.nt_idx * NT;
                    if (NT <= 64) slab16 = n_valid <= 8 ? 64u : (n_valid <= 16 ? 128u : (uint32_t)kSlab16);
                    // two issuers keep the tensor pipe, not the issuing thread, busy: a ragged tile then runs with a
                    // narrower MMA N (its rows rounded up to 32; the columns beyond it are never stored)
                    if (NT == 128 && TWO_ISSUERS && n_valid < NT) idesc = umma_idesc_bf16(kBlockM, (uint32_t)((n_valid + 31) & ~31));
                }
                {
                    XMOE_T0();
                    if (!mbar_wait(&acc_empty[as], aph ^ 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_EPI)) break;
                    XMOE_TACC(tw_acc);
                }
                tc_fence_after();
                const uint32_t acc = tmem_base + kAccBase + (as * kIssuers + issuer) * NT;
                uint32_t first = 1u;
                // this thread's K units of the segment: those whose CTA-wide number is `issuer` modulo kIssuers
                for (int ks = sg.ks0 + ((issuer - sg.it0) & (kIssuers - 1)); ks < sg.ks1; ks += kIssuers) {
                    const uint32_t it = (uint32_t)(sg.it0 + ks - sg.ks0);
                    const uint32_t bt = it / Cfg::kWUnits;  // token stage of this K unit
                    const uint32_t s = bt % kBStages, ph = (bt / kBStages) & 1u;
                    const uint32_t unit_slab = (it % Cfg::kWUnits) * Cfg::kSlabs;
                    const uint32_t d = it % kARing, dph = (it / kARing) & 1u;
                    {
                        XMOE_T0();
                        if (!mbar_wait(&b_full[s], ph, abort_flag, a.status, XMOE_DEV_TIMEOUT_TMA)) { ok = false; break; }
                        XMOE_TACC(tw_full);
                    }
                    const uint32_t a_tmem = tmem_base + d * kACols;
                    const uint32_t b_lo = b_lo0 + s * (uint32_t)(Cfg::kBStageBytes >> 4);
                    constexpr int kMmaPerPart = kStageK / 16 / Cfg::kSplit;
#pragma unroll
                    for (int part = 0; part < Cfg::kSplit; ++part) {
                        {
                            XMOE_T0();
                            if (!mbar_wait(&adq_full[d * Cfg::kSplit + part], dph, abort_flag, a.status, XMOE_DEV_TIMEOUT_DQ)) { ok = false; break; }
                            XMOE_TACC(tw_adq);
                        }
                        XMOE_T0();
                        tc_fence_after();
                        if (ks < k_stages) {  // a phantom stage only passes its slots on
#pragma unroll
                            for (int k2 = 0; k2 < kMmaPerPart; ++k2) {
                                const int kk = part * kMmaPerPart + k2;
                                // slab kk/4 (64 K each), 32 bytes of K per MMA inside the 128-byte swizzle row
                                mma_bf16_ts_lo(acc, a_tmem + kk * 8, b_lo + (unit_slab + (kk >> 2)) * slab16 + (kk & 3) * 2, idesc,
                                               (kk | (int)(first ^ 1u)) ? 1u : 0u);
                            }
                        }
                        tc_commit(&adq_empty[d * Cfg::kSplit + part]);
                        XMOE_TACC(t_issue);
                    }
                    if (!ok) break;
                    if (ks < k_stages) first = 0u;
                    tc_commit(&b_empty[s]);
                }
                if (ok) tc_commit(&acc_full[as]);
            }
            if (issuer == 0) {
                XMOE_TDUMP(2, tw_full);
                XMOE_TDUMP(3, tw_adq);
                XMOE_TDUMP(4, tw_acc);
                XMOE_TDUMP(5, t_issue);
            }
        }
    } else if (warp < 6) {
        // ------------------------------ epilogue -----------------------------------
        const int q = warp & 3;
        uint32_t tile_n = 0;
        uint16_t* out = reinterpret_cast<uint16_t*>(a.out);
        for (int si = 0; si < walk.n_seg; ++si, ++tile_n) {
            const KSegment sg = walk.seg(si, cta);
            const TileInfo t = tile_decode(sg.tile, prefix, a.counts, a.offsets, a.E_tot, NT);
            const uint32_t as = tile_n % kAccStages;
            const uint32_t aph = (tile_n / kAccStages) & 1u;
            if (!mbar_wait(&acc_full[as], aph, abort_flag, a.status, XMOE_DEV_TIMEOUT_ACC)) break;
            tc_fence_after();
            const int h_base = t.wt * kBlockM + q * 32;  // first feature of this warp's 32 lanes
            const int n_valid = min(NT, t.count - t.nt_idx * NT);
            const int real_units = min(sg.ks1, k_stages) - sg.ks0;  // K units of this segment that hold data
            const bool takes_partials = KSPLIT && sg.finishes && sg.ks0 > 0;  // other CTAs summed the K units before ks0
            const bool gives_partial = KSPLIT && !sg.finishes;                // this CTA only adds to the tile
            if (takes_partials) {
                // every helper's four epilogue warps have stored their quarter of the partial sum when its flag is 4
                if (lane == 0) {
                    for (int h = sg.first_helper; h < cta; ++h) {
                        uint32_t spin = 0;
                        while (ld_acquire_gpu(&a.split_flags[h]) < 4u) {
                            if (++spin > kPartialSpinLimit || *abort_flag) {
                                *abort_flag = 1u;
                                atomicCAS(a.status, XMOE_DEV_OK, XMOE_DEV_TIMEOUT_ACC | (blockIdx.x & 0xffu));
                                break;
                            }
                            __nanosleep(64);
                        }
                    }
                }
                __syncwarp();
            }
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + kAccBase + as * kIssuers * NT;
            for (int c0 = 0; c0 < NT; c0 += 32) {
                if (c0 >= n_valid) break;
                uint32_t v[32];
                unsigned long long my_row = 0ull;  // where token c0 + lane goes (0: nowhere)
                if (!gives_partial && c0 + lane < n_valid) {
                    const int prow = t.row0 + c0 + lane;
                    my_row = a.row_dst ? a.row_dst[prow] : (unsigned long long)(uintptr_t)(out + (size_t)prow * a.H);
                }
                // the segment's unit at offset o went to issuer (it0 + o) mod kIssuers: start from the issuer of
                // offset 0 (it always has data), then add the issuers of offsets 1, 2, 3 that exist
                const int p0 = sg.it0 & (kIssuers - 1);
                tmem_ld32(lane_addr + p0 * NT + c0, v);
                tmem_ld_wait();
                if (kIssuers > 1) {
#pragma unroll
                    for (int o = 1; o < kIssuers; ++o) {
                        if (o < real_units) {
                            const int p = (p0 + o) & (kIssuers - 1);
#pragma unroll
                            for (int hh = 0; hh < 2; ++hh) {  // 16 columns at a time: register budget
                                uint32_t v2[16];
                                tmem_ld16(lane_addr + p * NT + c0 + hh * 16, v2);
                                tmem_ld_wait();
#pragma unroll
                                for (int j = 0; j < 16; ++j)
                                    v[hh * 16 + j] =
                                        __float_as_uint(__uint_as_float(v[hh * 16 + j]) + __uint_as_float(v2[j]));
                            }
                        }
                    }
                }
                if (takes_partials) {  // helpers in CTA order (= K order), on top of this CTA's own sum
                    for (int h = sg.first_helper; h < cta; ++h) {
                        const float* part = a.split_partial + ((size_t)h * NT + c0) * kBlockM + q * 32 + lane;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (c0 + j < n_valid) v[j] = __float_as_uint(__uint_as_float(v[j]) + __ldcg(part + j * kBlockM));
                    }
                }
                if (gives_partial) {  // fp32, token-major: a warp writes 128 contiguous bytes per token
                    float* part = a.split_partial + ((size_t)cta * NT + c0) * kBlockM + q * 32 + lane;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (c0 + j < n_valid) part[j * kBlockM] = __uint_as_float(v[j]);
                    continue;
                }
                // lane = feature, v[j] = token c0 + j: store j of the warp writes 32 consecutive bf16 (64 bytes, two
                // whole sectors) of one output row. The row's home is this GPU's row buffer or (expert parallel) a
                // peer's return buffer; its address is fetched by the lane of the token's number and handed round.
                const int hf = h_base + lane;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const unsigned long long row = __shfl_sync(0xffffffffu, my_row, j);
                    if (row && hf < a.H)
                        reinterpret_cast<uint16_t*>((uintptr_t)row)[hf] = (uint16_t)f32_to_bf16_bits(__uint_as_float(v[j]));
                }
            }
            if (gives_partial) {  // publish: stores, fence, then this warp's count on the flag
                __threadfence();
                __syncwarp();
                if (lane == 0) atomicAdd(&a.split_flags[cta], 1u);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[as]);
        }
    } else {
        // ------------------------------ dequantiser --------------------------------
        // Tensor memory lanes are reachable per warp quadrant (warp index mod 4), so four
        // consecutive warps cover the 128 rows of a tile. kDqGroups such groups take the K
        // stages round-robin: expanding one stage is a serial chain of a few hundred
        // instructions per thread, and independent groups keep several stages in flight.
        const int quadrant = warp & 3;
        const int group = (warp - Cfg::kFirstDq) >> 2;
        const int row = quadrant * 32 + lane;
        // TMA swizzle of the raw tile: 128-byte rows -> chunk ^= row % 8; 64-byte rows -> chunk ^= (row / 2) % 4;
        // 32-byte rows -> chunk ^= (row / 4) % 2
        constexpr int kWRowBytes = Cfg::kWRowBytes;
        const uint32_t swz = kWRowBytes == 128 ? ((uint32_t)row & 7u)
                                               : (kWRowBytes == 64 ? ((uint32_t)(row >> 1) & 3u) : ((uint32_t)(row >> 2) & 1u));
        const __nv_bfloat162 bias = bf162_from_bits(0x43084308u);  // 136.0 twice
        long long dq_wfull = 0, dq_wempty = 0, dq_work = 0;  // dq_work includes the wait for the slot
        (void)dq_wfull; (void)dq_wempty; (void)dq_work;
        // The K stages of all tiles of this CTA are numbered through (it, k_walk slots per tile); this group
        // takes it = group, group + kDqGroups, ... Everything that follows from `it` is kept incrementally:
        // the tensor-memory slot is always `group` (kARing == kDqGroups or a multiple handled below), the
        // weight stage advances by kDqGroups / kWUnits slots per step and the K unit inside it never changes.
        uint32_t total_it = 0;
        for (int si = 0; si < walk.n_seg; ++si) {
            const KSegment g = walk.seg(si, cta);
            total_it += (uint32_t)(g.ks1 - g.ks0);
        }
        int seg_i = 0;
        KSegment sg = walk.seg(0, cta);  // segment that holds unit `it` (n_seg == 0: never used)
        const uint32_t w_base_u32 = smem_u32(w_base);
        constexpr int kWStep = kDqGroups / Cfg::kWUnits;        // weight stages per step of this group
        const int unit = group % Cfg::kWUnits;                  // which K unit of the weight stage (k_walk is a multiple of kWUnits)
        int s = (group / Cfg::kWUnits) % kWStages;              // weight slot of stage `it`
        uint32_t ph = 0;
        int d = group % kARing;
        uint32_t dph = 0;
#ifdef XMOE_TRACE
        const long long dq_t_begin = clock64();
#endif
        const uint32_t row_off = (uint32_t)row * kWRowBytes;
        const uint32_t scale_off = Cfg::kWRawBytes + unit * 256 + row * 2;
        const uint32_t a_lane0 = tmem_base + ((uint32_t)(quadrant * 32) << 16);
        for (uint32_t it = (uint32_t)group; it < total_it; it += kDqGroups) {
            while ((int)it >= sg.it0 + (sg.ks1 - sg.ks0)) sg = walk.seg(++seg_i, cta);
            const int ks = sg.ks0 + ((int)it - sg.it0);
            {
                XMOE_T0();
                if (!mbar_wait(&w_full[s], ph, abort_flag, a.status, XMOE_DEV_TIMEOUT_TMA)) break;
                XMOE_TACC(dq_wfull);
            }
            XMOE_T0();
            if (ks >= k_stages) {
                // phantom stage (odd K-unit count): keep this group's place in both rings, expand nothing
                bool ok = true;
#pragma unroll
                for (int part = 0; part < Cfg::kSplit; ++part)
                    ok = ok && mbar_wait(&adq_empty[d * Cfg::kSplit + part], dph ^ 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_DQ);
                if (!ok) break;
                __syncwarp();
                if (lane == 0) {
#pragma unroll
                    for (int part = 0; part < Cfg::kSplit; ++part) mbar_arrive(&adq_full[d * Cfg::kSplit + part]);
                }
            } else {
                const uint32_t st = w_base_u32 + (uint32_t)s * Cfg::kWStageBytes;
                const uint32_t sraw = lds_u16(st + scale_off);
                const __nv_bfloat162 s2 = bf162_from_bits(__byte_perm(sraw, sraw, 0x1010));
                const uint32_t a_lane = a_lane0 + d * kACols;
                bool ok = true;
                // 16 bytes (32 weights) at a time: four words -> sixteen bf16x2 registers -> one 16-column store
                constexpr int kChunksPerPart = kStageK / 32 / Cfg::kSplit;
                // all of the row's 16-byte pieces first (independent loads in flight together: with one load per
                // piece the warps stalled on the shared-memory scoreboard for a third of their issue cycles)
                uint4 raw[kStageK / 32];
#pragma unroll
                for (int q = 0; q < kStageK / 32; ++q)
                    raw[q] = lds_u128(st + row_off + (((uint32_t)(unit * (kStageK / 32) + q) ^ swz) * 16));
#pragma unroll
                for (int q = 0; q < kStageK / 32; ++q) {
                    const int part = q / kChunksPerPart;
                    const uint4 r4 = raw[q];
                    uint32_t o[16];
                    expand_word(r4.x, o, bias, s2);
                    expand_word(r4.y, o + 4, bias, s2);
                    expand_word(r4.z, o + 8, bias, s2);
                    expand_word(r4.w, o + 12, bias, s2);
                    if (q % kChunksPerPart == 0) {
                        // the expansion above does not need the tensor-memory slot: wait for it only now
                        XMOE_T1();
                        if (!mbar_wait(&adq_empty[d * Cfg::kSplit + part], dph ^ 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_DQ)) { ok = false; break; }
                        XMOE_TACC1(dq_wempty);
                        tc_fence_after();
                    }
                    tmem_st16(a_lane + q * 16, o);
                    if (q % kChunksPerPart == kChunksPerPart - 1) {  // this part is complete: hand it to the issuer
                        tmem_st_wait();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&adq_full[d * Cfg::kSplit + part]);
                    }
                }
                if (!ok) break;
            }
            if (lane == 0) mbar_arrive(&w_empty[s]);
            XMOE_TACC(dq_work);
            s += kWStep;
            if (s >= kWStages) { s -= kWStages; ph ^= 1u; }
            if (kARing == kDqGroups) {
                dph ^= 1u;
            } else {
                d += kDqGroups;
                if (d >= kARing) { d -= kARing; dph ^= 1u; }
            }
        }
        if (warp == Cfg::kFirstDq && lane == 0) {
            XMOE_TDUMP(6, dq_wfull);
            XMOE_TDUMP(7, dq_wempty);
            XMOE_TDUMP(8, dq_work);
#ifdef XMOE_TRACE
            XMOE_TDUMP(9, clock64() - dq_t_begin);
            XMOE_TDUMP(10, (long long)total_it);
#endif
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

template <int NT, bool KSPLIT, bool TWO_ISSUERS = false>
int launch_ff2_nt(const Ff2Args& a, cudaStream_t stream) {
    using Cfg = Ff2Cfg<NT, TWO_ISSUERS>;
    static bool attr_set_dev[kMaxDevices] = {};
    const int dev = device_slot();
    if (dev < 0) return XMOE_ERR_CUDA;
    bool& attr_set = attr_set_dev[dev];
    if (!attr_set) {
        if (cudaFuncSetAttribute(ff2_w4a16_kernel<NT, KSPLIT, TWO_ISSUERS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)Cfg::kSmemBytes) != cudaSuccess)
            return XMOE_ERR_CUDA;
        attr_set = true;
    }
    ff2_w4a16_kernel<NT, KSPLIT, TWO_ISSUERS><<<a.num_sms, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(a);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

}  // namespace

#ifdef XMOE_TRACE
extern "C" int xmoe_ff2_trace_dump(long long* host_out) {
    return (int)cudaMemcpyFromSymbol(host_out, g_ff2_trace, sizeof(g_ff2_trace));
}
#endif

int launch_ff2(const Ff2Args& a, cudaStream_t stream) {
    if (a.E_tot + 1 > kMaxExperts || a.H % 8 || a.I % 32) return XMOE_ERR_SHAPE;
    const bool split = a.split_partial != nullptr && a.split_flags != nullptr;
    // K lengths (in units of 128) at which the two-issuer variants take over; the environment variables are for
    // measurements
    static const int small_two_max = [] { const char* e = getenv("XMOE_FF2_SMALL_TWO_MAX_GROUPS"); return e ? atoi(e) : 7; }();
    static const int t128_two_min = [] { const char* e = getenv("XMOE_FF2_T128_TWO_MIN_GROUPS"); return e ? atoi(e) : 12; }();
    switch (a.nt) {
        // Small token tiles: four issuing threads (one accumulator set for 64 tokens, two for 32), or two issuing
        // threads with twice the accumulator sets when K is short (<= 7 units): the epilogue then adds two partial
        // sums instead of four, and with tiles of a few units it, not the MMAs, sets the pace (Qwen3 shape, 6 units,
        // 512 tokens: 73 -> 55 us; with 8 units per tile two threads are 6 % slower than four, with 23 or 112 units 5-13 %).
        case 32:
            if (a.groups <= small_two_max) return launch_ff2_nt<32, false, true>(a, stream);
            return split ? launch_ff2_nt<32, true>(a, stream) : launch_ff2_nt<32, false>(a, stream);
        case 64:
            if (a.groups <= small_two_max) return launch_ff2_nt<64, false, true>(a, stream);
            return split ? launch_ff2_nt<64, true>(a, stream) : launch_ff2_nt<64, false>(a, stream);
        // 128-token tiles: with a long K (>= 12 units) two issuing threads, each with its own accumulator, beat one
        // thread with two accumulator sets (DeepSeek-V3 shape, 16 units: 917 against 970-1020 us at 2048 tokens, 704
        // against 994 us at 256); with a short K the overlapped epilogue wins (Qwen3 shape, 6 units: 275 against 383 us)
        case 128: return a.groups >= t128_two_min ? launch_ff2_nt<128, false, true>(a, stream) : launch_ff2_nt<128, false>(a, stream);
        case 256: return launch_ff2_nt<256, false>(a, stream);
        default: return XMOE_ERR_SHAPE;
    }
}

}  // namespace xmoe
