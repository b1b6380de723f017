// FF2: grouped W4A16 down projection. int4 group-128 weights are expanded to bf16 in
// shared memory ahead of a bf16 tcgen05 MMA; activations are the bf16 FF1 output.
//
// Weight contract: symmetric int4, group 128 along K, w = (u4 - 8) * scale[k/128] -- the
// GPTQ / compressed-tensors contract of the reference's INT4 lane
// (xFused-XXXX-Kernels/xMoE/xW4A16/sm75/xR64/xR64ABSRepack.cu:3-24, xR64ABS.cuh:30-34,
// vllm/xcaliber_int4_vllm/method.py:188-203). The "expand 4-bit weights with a few
// logic ops, then use the 16-bit tensor path" idea is the one the reference sketches in
// xFused-NVFP4-Kernels/ptx.cuh:1-83; the expansion here is the integer flavour:
// (nibble | 0x4300) is the bf16 value 128 + nibble, minus 136 gives nibble - 8 exactly,
// one bf16x2 multiply applies the group scale (one rounding, same as bf16(w * s)).
//
// Structure (swap-AB like FF1: 128 output features = MMA M, NT tokens = MMA N):
//   warp 0      TMA producer: raw int4 tile (128 rows x 64 B = K 128), its 128 bf16 group
//               scales, and the bf16 activation tile (NT rows x K 128, 128-byte swizzle)
//   warps 6-13  dequantise the raw tile into a K-major 128-byte-swizzled bf16 tile
//               (two 64-K slabs), fence to the async proxy, signal the MMA warp
//   warp 1      tcgen05.mma kind::f16 (bf16 x bf16 -> fp32 in TMEM), K = 16 per instruction
//   warps 2-5   epilogue: tcgen05.ld -> bf16 rows [packed row, H]
// One K stage is exactly one quantisation group, so a row needs one scale per stage.
#include <cuda_bf16.h>

#include "common.cuh"
#include "kernels.h"

namespace xmoe {

namespace {

constexpr int kBlockM = 128;
constexpr int kStageK = 128;                     // one int4 group
constexpr int kRawBytes = kBlockM * kStageK / 2; // 8 KiB
constexpr int kScaleBytes = kBlockM * 2;         // 256 B
constexpr int kADqBytes = kBlockM * kStageK * 2; // 32 KiB = two 16 KiB slabs
constexpr int kDqWarps = 8;
constexpr int kThreads = 32 * (6 + kDqWarps);    // 448
constexpr int kMaxExperts = 1024 + 8;
constexpr int kTmemCols = 256;

template <int NT>
struct Ff2Cfg {
    static constexpr int kBBytes = NT * kStageK * 2;        // two slabs of NT x 128 B
    static constexpr int kStageBytes = kRawBytes + 1024 /*scales, padded*/ + kBBytes;
    static constexpr int kStages = NT >= 128 ? 3 : (NT >= 64 ? 3 : 5);
    static constexpr int kADqStages = NT >= 128 ? 3 : 4;  // bf16 weight tiles in flight between dequant and MMA
    static constexpr int kAccStages = 2;
    static_assert(kAccStages * NT <= kTmemCols, "TMEM budget");
    static constexpr int kTxBytes = kRawBytes + kScaleBytes + kBBytes;
    static constexpr size_t kSmemBytes =
        1024 + (size_t)kStages * kStageBytes + (size_t)kADqStages * kADqBytes + 5120;
};

struct TileInfo {
    int e, mt, nt_idx, count, row0;
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

__device__ __forceinline__ void build_tile_prefix(int* prefix, const int32_t* counts, int e_tot, int mt_tiles, int NT) {
    const int lane = threadIdx.x & 31;
    int carry = 0;
    for (int base = 0; base < e_tot; base += 32) {
        const int e = base + lane;
        const int v = e < e_tot ? ((counts[e] + NT - 1) / NT) * mt_tiles : 0;
        int incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += o;
        }
        if (e < e_tot) prefix[e] = carry + incl - v;
        carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) prefix[e_tot] = carry;
}

__device__ __forceinline__ TileInfo decode_tile(int item, const int* prefix, const int32_t* counts,
                                                const int32_t* offsets, int e_tot, int NT) {
    int lo = 0, hi = e_tot;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (prefix[mid] <= item) lo = mid; else hi = mid;
    }
    TileInfo t;
    t.e = lo;
    const int local = item - prefix[lo];
    t.count = counts[lo];
    const int n_tiles = (t.count + NT - 1) / NT;
    t.mt = local / n_tiles;
    t.nt_idx = local % n_tiles;
    t.row0 = offsets[lo] + t.nt_idx * NT;
    return t;
}

template <int NT>
__global__ __launch_bounds__(kThreads, 1) void ff2_w4a16_kernel(const __grid_constant__ Ff2Args a) {
    using Cfg = Ff2Cfg<NT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* stage_base = smem;
    uint8_t* adq_base = smem + (size_t)Cfg::kStages * Cfg::kStageBytes;
    uint8_t* tail = adq_base + (size_t)Cfg::kADqStages * kADqBytes;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);  // [kStages]   TMA landed
    uint64_t* empty_bar = full_bar + 8;                      // [kStages]   dequant warps + MMA done with the stage
    uint64_t* adq_full = empty_bar + 8;                      // [4]         bf16 weight tile ready
    uint64_t* adq_empty = adq_full + 4;                      // [4]         MMAs reading it retired
    uint64_t* acc_full = adq_empty + 4;                      // [2]
    uint64_t* acc_empty = acc_full + 2;                      // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    int* prefix = reinterpret_cast<int*>(tail + 256);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int mt_tiles = (a.H + kBlockM - 1) / kBlockM;
    const int k_stages = a.groups;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], kDqWarps + 1);
        }
        for (int s = 0; s < Cfg::kADqStages; ++s) {
            mbar_init(&adq_full[s], kDqWarps);
            mbar_init(&adq_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 4);
        }
        *abort_flag = 0u;
        mbar_fence_init();
        prefetch_tmap(&a.tm_w);
        prefetch_tmap(&a.tm_y);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    if (warp == 2) build_tile_prefix(prefix, a.counts, a.E_tot, mt_tiles, NT);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int total_tiles = prefix[a.E_tot];

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            const uint16_t* scales = reinterpret_cast<const uint16_t*>(a.w2_scale);
            uint32_t it = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < total_tiles && ok; item += gridDim.x) {
                const TileInfo t = decode_tile(item, prefix, a.counts, a.offsets, a.E_tot, NT);
                const int h0 = t.mt * kBlockM;
                const int w_row = t.e * a.H + h0;
                const int rows_here = min(kBlockM, a.H - h0);
                const uint32_t scale_bytes = (uint32_t)rows_here * 2u;  // H % 8 == 0 keeps this a multiple of 16
                for (int ks = 0; ks < k_stages; ++ks, ++it) {
                    const int s = it % Cfg::kStages;
                    const uint32_t ph = (it / Cfg::kStages) & 1u;
                    if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_MMA)) {
                        ok = false;
                        break;
                    }
                    uint8_t* st = stage_base + (size_t)s * Cfg::kStageBytes;
                    mbar_expect_tx(&full_bar[s], kRawBytes + scale_bytes + Cfg::kBBytes);
                    tma_load_2d(st, &a.tm_w, ks * (kStageK / 2), w_row, &full_bar[s]);
                    tma_load_1d(st + kRawBytes, scales + ((size_t)t.e * a.groups + ks) * a.H + h0, scale_bytes,
                                &full_bar[s]);
                    uint8_t* b = st + kRawBytes + 1024;
                    tma_load_2d(b, &a.tm_y, ks * kStageK, t.row0, &full_bar[s]);
                    tma_load_2d(b + NT * 128, &a.tm_y, ks * kStageK + 64, t.row0, &full_bar[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(kBlockM, NT);
            uint32_t it = 0, tile_n = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < total_tiles && ok; item += gridDim.x, ++tile_n) {
                const uint32_t as = tile_n & 1u;
                const uint32_t aph = (tile_n >> 1) & 1u;
                if (!mbar_wait(&acc_empty[as], aph ^ 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_EPI)) break;
                tc_fence_after();
                const uint32_t acc = tmem_base + as * NT;
                for (int ks = 0; ks < k_stages; ++ks, ++it) {
                    const int s = it % Cfg::kStages;
                    const uint32_t ph = (it / Cfg::kStages) & 1u;
                    const int d = it % Cfg::kADqStages;
                    const uint32_t dph = (it / Cfg::kADqStages) & 1u;
                    if (!mbar_wait(&full_bar[s], ph, abort_flag, a.status, XMOE_DEV_TIMEOUT_TMA) ||
                        !mbar_wait(&adq_full[d], dph, abort_flag, a.status, XMOE_DEV_TIMEOUT_DQ)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_smem = smem_u32(adq_base + (size_t)d * kADqBytes);
                    const uint32_t b_smem = smem_u32(stage_base + (size_t)s * Cfg::kStageBytes + kRawBytes + 1024);
#pragma unroll
                    for (int kk = 0; kk < kStageK / 16; ++kk) {
                        const int slab = kk >> 2;
                        const uint64_t koff = (uint64_t)(((kk & 3) * 32) >> 4);
                        const uint64_t da = umma_desc_sw128(a_smem + slab * (kBlockM * 128)) + koff;
                        const uint64_t db = umma_desc_sw128(b_smem + slab * (NT * 128)) + koff;
                        mma_bf16(acc, da, db, idesc, (ks | kk) ? 1u : 0u);
                    }
                    tc_commit(&empty_bar[s]);
                    tc_commit(&adq_empty[d]);
                }
                if (ok) tc_commit(&acc_full[as]);
            }
        }
    } else if (warp < 6) {
        // ------------------------------ epilogue -----------------------------------
        const int q = warp & 3;
        uint32_t tile_n = 0;
        uint16_t* out = reinterpret_cast<uint16_t*>(a.out);
        for (int item = blockIdx.x; item < total_tiles; item += gridDim.x, ++tile_n) {
            const TileInfo t = decode_tile(item, prefix, a.counts, a.offsets, a.E_tot, NT);
            const uint32_t as = tile_n & 1u;
            const uint32_t aph = (tile_n >> 1) & 1u;
            if (!mbar_wait(&acc_full[as], aph, abort_flag, a.status, XMOE_DEV_TIMEOUT_ACC)) break;
            tc_fence_after();
            const int h_idx = t.mt * kBlockM + q * 32 + lane;
            const bool h_ok = h_idx < a.H;
            const int n_valid = min(NT, t.count - t.nt_idx * NT);
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + as * NT;
            for (int c0 = 0; c0 < NT; c0 += 32) {
                if (c0 >= n_valid) break;
                uint32_t v[32];
                tmem_ld32(lane_addr + c0, v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int n = c0 + j;
                    if (n < n_valid && h_ok)
                        out[(size_t)(t.row0 + n) * a.H + h_idx] = (uint16_t)f32_to_bf16_bits(__uint_as_float(v[j]));
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[as]);
        }
    } else {
        // ------------------------------ dequantiser --------------------------------
        const int dq_tid = threadIdx.x - 6 * 32;  // 0..255
        uint32_t it = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < total_tiles && ok; item += gridDim.x) {
            for (int ks = 0; ks < k_stages; ++ks, ++it) {
                const int s = it % Cfg::kStages;
                const uint32_t ph = (it / Cfg::kStages) & 1u;
                const int d = it % Cfg::kADqStages;
                const uint32_t dph = (it / Cfg::kADqStages) & 1u;
                if (!mbar_wait(&full_bar[s], ph, abort_flag, a.status, XMOE_DEV_TIMEOUT_TMA) ||
                    !mbar_wait(&adq_empty[d], dph ^ 1u, abort_flag, a.status, XMOE_DEV_TIMEOUT_DQ)) {
                    ok = false;
                    break;
                }
                const uint8_t* st = stage_base + (size_t)s * Cfg::kStageBytes;
                const uint4* raw = reinterpret_cast<const uint4*>(st);
                const uint16_t* sc = reinterpret_cast<const uint16_t*>(st + kRawBytes);
                uint8_t* dst = adq_base + (size_t)d * kADqBytes;
#pragma unroll
                for (int rep = 0; rep < 2; ++rep) {
                    const int c = dq_tid + rep * 256;  // 16-byte chunk of the raw tile
                    const int row = c >> 2, part = c & 3;
                    const uint4 r4 = raw[c];
                    const uint32_t words[4] = {r4.x, r4.y, r4.z, r4.w};
                    const uint32_t sraw = sc[row];
                    const __nv_bfloat162 s2 = bf162_from_bits(sraw | (sraw << 16));
                    const __nv_bfloat162 bias = bf162_from_bits(0x43084308u);  // 136.0 twice
                    uint8_t* slab = dst + (part >> 1) * (kBlockM * 128) + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        uint32_t o[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t bits = ((words[w] >> (4 * j)) & 0x000f000fu) | 0x43004300u;
                            o[j] = bits_from_bf162(__hmul2(__hsub2(bf162_from_bits(bits), bias), s2));
                        }
                        const int chunk = (part & 1) * 4 + w;  // 16-byte chunk inside the 128-byte row
                        *reinterpret_cast<uint4*>(slab + ((chunk ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&adq_full[d]);
                    mbar_arrive(&empty_bar[s]);
                }
            }
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

template <int NT>
int launch_ff2_nt(const Ff2Args& a, cudaStream_t stream) {
    using Cfg = Ff2Cfg<NT>;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(ff2_w4a16_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)Cfg::kSmemBytes) != cudaSuccess)
            return XMOE_ERR_CUDA;
        attr_set = true;
    }
    ff2_w4a16_kernel<NT><<<a.num_sms, kThreads, Cfg::kSmemBytes, stream>>>(a);
    return cudaGetLastError() == cudaSuccess ? XMOE_OK : XMOE_ERR_CUDA;
}

}  // namespace

int launch_ff2(const Ff2Args& a, cudaStream_t stream) {
    if (a.E_tot + 1 > kMaxExperts || a.H % 8 || a.I % 32) return XMOE_ERR_SHAPE;
    switch (a.nt) {
        case 32: return launch_ff2_nt<32>(a, stream);
        case 64: return launch_ff2_nt<64>(a, stream);
        case 128: return launch_ff2_nt<128>(a, stream);
        default: return XMOE_ERR_SHAPE;
    }
}

}  // namespace xmoe
