// C ABI of the fused MoE layer: argument checks, workspace carving, TMA tensor-map
// encoding, and the stage sequence. Mirrors the role of the reference bridge
// (xFused-XXXX-Kernels/xMoE/xW4A16/sm75/xR64/vllm/csrc/xr64_abs_bridge.cu:81-232) with
// two differences: scratch is caller-owned instead of torch::empty per call, and
// errors come back as status codes instead of TORCH_CHECK exceptions.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/xmoe_b200.h"
#include "common.cuh"
#include "kernels.h"

using namespace xmoe;

#define XMOE_STR2(x) #x
#define XMOE_STR(x) XMOE_STR2(x)

namespace {

// ---- driver entry point for tensor-map encoding (no link-time libcuda dependency) -----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
    return fn;
}

// 2-D row-major tensor [rows, inner] of `elem_bytes` elements, box [box_rows, box_inner].
int make_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t inner,
                 uint64_t rows, uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swz) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return XMOE_ERR_CUDA;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || ((inner * elem_bytes) & 15u)) return XMOE_ERR_SHAPE;
    cuuint64_t dims[2] = {inner, rows};
    cuuint64_t strides[1] = {inner * (uint64_t)elem_bytes};
    cuuint32_t box[2] = {box_inner, box_rows};
    cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? XMOE_OK : XMOE_ERR_CUDA;
}

// The same row-major tensor [rows, inner] seen as [inner / 64][rows][64] (inner % 64 == 0): box [kblocks][box_rows][64].
// One copy then lands `kblocks` consecutive 128-byte-swizzle slabs of box_rows x 64 elements.
int make_tmap_kslabs(CUtensorMap* out, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t inner,
                     uint64_t rows, uint32_t box_rows, uint32_t kblocks) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return XMOE_ERR_CUDA;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || ((inner * elem_bytes) & 15u) || inner % 64) return XMOE_ERR_SHAPE;
    cuuint64_t dims[3] = {64, rows, inner / 64};
    cuuint64_t strides[2] = {inner * (uint64_t)elem_bytes, 64 * (uint64_t)elem_bytes};
    cuuint32_t box[3] = {64, box_rows, kblocks};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? XMOE_OK : XMOE_ERR_CUDA;
}

int num_sms() {  // of the current device
    static int n_dev[kMaxDevices] = {};
    const int dev = device_slot();
    if (dev < 0) return 148;
    int& n = n_dev[dev];
    if (!n && (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)) n = 148;
    return n;
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// The activation amax pass does not depend on routing: it runs on a side stream of the library,
// forked after the scalar block is cleared and joined before the quantiser, so that it overlaps the
// router and the route pack (the reference plans the same overlap with CUDA-graph child graphs,
// co-design.md:132-158). One non-blocking stream and two events per device, created on first use
// outside stream capture; XMOE_FORK=0 keeps everything on the caller's stream.
struct SideStream {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
};
SideStream* side_stream(cudaStream_t caller) {
    static const bool enabled = [] {
        const char* e = getenv("XMOE_FORK");
        return !(e && e[0] == '0');
    }();
    if (!enabled) return nullptr;
    static SideStream per_device[kMaxDevices];
    static std::mutex mu;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    SideStream& s = per_device[dev];
    if (!s.stream) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(caller, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return nullptr;
        if (cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming) != cudaSuccess) {
            s = SideStream();
            return nullptr;
        }
    }
    return &s;
}

// The first 4 KiB of a workspace are cleared at the start of every call. The first KiB holds scalars: status
// word of the layer (word 0), amax scratch, activation scale; word 32 is the status of the gate GEMM when
// xmoe_forward_gated runs it. The host_io workspace of xmoe_forward_host is read the same way (its gate word
// is never written and stays as allocated: zeroed here). Bytes 1024.. hold the per-CTA flags of FF2's
// K-split partial sums (zero at launch).
constexpr int kGateStatusWord = 32;
constexpr size_t kClearedBytes = 4096;
constexpr size_t kFf2FlagsOffset = 1024;
constexpr int kMaxSplitCtas = 192;  // flag words and partial-sum slots reserved (B200: 148 SMs)
static_assert(kFf2FlagsOffset + kMaxSplitCtas * 4 <= 2048, "flag block");

// ---- optional per-stage timing (CUDA events recorded on the caller's stream) -----------
constexpr int kProfStages = 8;  // router, pack, amax, quant, ff1, act_topk, ff2, combine
struct Profiler {
    cudaEvent_t* ev = nullptr;  // [max_steps][kProfStages + 1]
    int max_steps = 0;
    int step = 0;
} g_prof;

inline void prof_mark(int stage_boundary, cudaStream_t s) {
    if (g_prof.ev && g_prof.step < g_prof.max_steps)
        cudaEventRecord(g_prof.ev[(size_t)g_prof.step * (kProfStages + 1) + stage_boundary], s);
}

int check_cfg(const xmoe_config* c) {
    if (!c) return XMOE_ERR_ARG;
    if (c->hidden <= 0 || c->inter <= 0 || c->num_experts <= 0 || c->top_k <= 0) return XMOE_ERR_ARG;
    if (c->hidden % 64 || c->inter % 32) return XMOE_ERR_SHAPE;
    if (c->num_experts > 1024 || c->top_k > 8 || c->top_k > c->num_experts) return XMOE_ERR_SHAPE;
    if (c->num_shared_experts < 0 || c->num_shared_experts > 8) return XMOE_ERR_SHAPE;
    if (c->scoring < 0 || c->scoring > 1 || c->activation < 0 || c->activation > 2) return XMOE_ERR_SHAPE;
    if (c->n_group < 0 || c->n_group > 32) return XMOE_ERR_SHAPE;
    if (c->token_tile != 0 && c->token_tile != 32 && c->token_tile != 64 && c->token_tile != 128)
        return XMOE_ERR_SHAPE;
    if (c->act_topk_keep < 0 || c->act_topk_keep > c->inter) return XMOE_ERR_SHAPE;
    return XMOE_OK;
}

// Token tile of a call (rows of every expert are padded to it): 128 once the routed experts hold about 24 rows each on
// average, 32 below that. Shared experts take every token, but they are few: the routed experts decide. Measured on
// one B200, layer time in us with tiles 32 / 64 / 128 (the 64-token tile never won; it stays selectable through
// xmoe_config.token_tile): Mixtral shape 64 tokens (16 rows per expert) 201 / 221 / 221, 128 tokens (32) 233 / 214 /
// 212; gpt-oss 512 tokens (16) 393 / 430 / 425, 1024 (32) 479 / 455 / 441; Qwen3 512 tokens (32) 147 / 139 / 117;
// DeepSeek-V3 shape 512 tokens (16 routed) 1379 / 1490 / 1528, 1024 (32) 1800 / 1673 / 1607.
int pick_token_tile(const xmoe_config* c, int n) {
    if (c->token_tile) return c->token_tile;
    const double avg_routed = (double)n * c->top_k / c->num_experts;
    return avg_routed >= 24.0 ? 128 : 32;
}

// FF2 may use a wider token tile than FF1: the 256-token tile (CTA pairs) keeps the bf16 pipe at its full rate
// (an N = 128 MMA is bound by the issuing thread, not by the pipe), but its accumulator is single, so the
// epilogue is not overlapped: it pays with a long K (I >= min_inter) and with experts that fill the tile
// (average rows per expert >= min_rows = 112; FF2 time in us, pair against single-CTA kernel: gpt-oss shape at 96 rows
// per expert 323 / 257, at 128 rows 351 / 364; Mixtral shape at 128 rows 145 / 150, at 192 rows 161 / 196; DeepSeek-V3
// shape at 72 rows 1050 / 845, at 143 rows 1275 / 1503). `rows_in_use` = N * k_eff.
int ff2_token_tile(const xmoe_config* c, int nt, size_t rows_in_use) {
    static const int min_inter = [] { const char* e = getenv("XMOE_FF2_T256_MIN_INTER"); return e ? atoi(e) : 2048; }();
    static const int min_rows = [] { const char* e = getenv("XMOE_FF2_T256_MIN_ROWS"); return e ? atoi(e) : 112; }();
    const size_t e_tot = (size_t)c->num_experts + c->num_shared_experts;
    // a short K (inter < min_inter) pays only with experts that fill the 256-token tiles several times over (Qwen3
    // shape, 6 K units: 257 against 273 us at 512 rows per expert, 110 against 101 us at 128)
    const size_t need = c->inter >= min_inter ? (size_t)min_rows : (size_t)384;
    return (nt == 128 && rows_in_use >= need * e_tot) ? 256 : nt;
}

struct Layout {
    int k_eff, e_tot, kb_pad, mb, groups, nt, chunks;
    size_t rows;  // packed-row capacity
    size_t off_status, off_amax, off_scale, off_topk_idx, off_topk_w, off_topk_off, off_topk_row, off_hist, off_counts,
        off_offsets, off_row_token, off_row_weight, off_xq, off_sfx, off_yact, off_out, off_ff2_partial, off_row_dst, total;
    size_t off_x_in, off_logits_in, off_y_out, total_host_io;
};

size_t packed_rows(const xmoe_config* c, int n) {
    const size_t k_eff = (size_t)c->top_k + c->num_shared_experts;
    const size_t e_tot = (size_t)c->num_experts + c->num_shared_experts;
    const size_t assign = (size_t)n * k_eff;
    const size_t live = assign < e_tot ? assign : e_tot;
    return align_up(assign + live * 127, 128);
}

Layout make_layout(const xmoe_config* c, int n) {
    Layout L;
    L.k_eff = c->top_k + c->num_shared_experts;
    L.e_tot = c->num_experts + c->num_shared_experts;
    L.kb_pad = (int)align_up((size_t)c->hidden / 64, 4);
    L.mb = (c->inter + 127) / 128;
    L.groups = (c->inter + 127) / 128;
    L.nt = pick_token_tile(c, n);
    L.chunks = route_pack_chunks(n > 0 ? n : 1);
    L.rows = packed_rows(c, n);
    size_t o = 0;
    auto take = [&](size_t bytes) {
        const size_t at = o;
        o = align_up(o + bytes, 1024);
        return at;
    };
    L.off_status = take(kClearedBytes);  // status word, scalars and flags (see kClearedBytes)
    L.off_amax = 16;
    L.off_scale = 32;
    L.off_topk_idx = take((size_t)n * L.k_eff * 4);
    L.off_topk_w = take((size_t)n * L.k_eff * 2);
    L.off_topk_off = take((size_t)n * L.k_eff * 4);
    L.off_topk_row = take((size_t)n * L.k_eff * 4);
    L.off_hist = take((size_t)L.chunks * L.e_tot * 4);
    L.off_counts = take((size_t)L.e_tot * 4);
    L.off_offsets = take((size_t)(L.e_tot + 1) * 4);
    L.off_row_token = take(L.rows * 4);
    L.off_row_weight = take(L.rows * 2);
    L.off_xq = take(L.rows * (size_t)(c->hidden / 2));
    L.off_sfx = take((L.rows / L.nt) * (size_t)L.kb_pad * 512);
    L.off_yact = take(L.rows * (size_t)c->inter * 2);
    L.off_out = take(L.rows * (size_t)c->hidden * 2);
    // small token tiles: one fp32 partial-sum slot [token tile][128] per CTA for FF2's K split
    L.off_ff2_partial = take(L.nt <= 64 ? (size_t)kMaxSplitCtas * 64 * 128 * 4 : 0);
    L.off_row_dst = take(L.rows * 8);  // per-row destinations of xmoe_forward_routed_scatter
    L.total = o;
    L.off_x_in = take((size_t)n * c->hidden * 2);
    L.off_logits_in = take((size_t)n * c->num_experts * 2);
    L.off_y_out = take((size_t)n * c->hidden * 2);
    L.total_host_io = o;
    return L;
}

int run_ff1(const void* w13_packed, const void* w13_sf, const float* w13_gs, const void* xq, const void* sfx,
            const float* act_scale, const int32_t* counts, const int32_t* offsets, const void* row_weight, void* yact,
            uint32_t* status, int e_tot, int H, int I, size_t rows, int nt, int activation, float alpha, float limit,
            cudaStream_t stream) {
    Ff1Args a;
    memset(&a, 0, sizeof(a));
    int rc = make_tmap_2d(&a.tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w13_packed, (uint64_t)H / 2,
                          (uint64_t)e_tot * 2 * I, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_tmap_2d(&a.tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, (uint64_t)H / 2, rows, 128, (uint32_t)nt,
                      CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    a.sfw = (const uint8_t*)w13_sf;
    a.sfx = (const uint8_t*)sfx;
    a.w13_gs = w13_gs;
    a.scale = (const ActScale*)act_scale;
    a.counts = counts;
    a.offsets = offsets;
    a.row_weight = row_weight;
    a.yact = yact;
    a.status = status;
    a.E_tot = e_tot;
    a.H = H;
    a.I = I;
    a.kb_pad = (int)align_up((size_t)H / 64, 4);
    a.mb = (I + 127) / 128;
    a.nt = nt;
    a.activation = activation;
    a.alpha = alpha;
    a.limit = limit;
    a.num_sms = num_sms();
    // prefill-sized experts run 256-token tiles on CTA pairs unless XMOE_FF1_PAIR=0
    const char* pair_env = getenv("XMOE_FF1_PAIR");
    const bool pair_enabled = !(pair_env && pair_env[0] == '0');
    static const size_t pair_min_rows = [] { const char* e = getenv("XMOE_FF1_PAIR_MIN_ROWS"); return (size_t)(e ? atoi(e) : 320); }();
    if (nt == 128 && pair_enabled && a.num_sms >= 2 && rows / (size_t)e_tot >= pair_min_rows) return launch_ff1_pair(a, stream);
    return launch_ff1(a, stream);
}

int run_ff2(const void* w2_q, const void* w2_scale, const void* yact, const int32_t* counts, const int32_t* offsets,
            void* out_rows, uint32_t* status, int e_tot, int H, int I, size_t rows, int nt, cudaStream_t stream,
            const unsigned long long* row_dst = nullptr, float* split_partial = nullptr, uint32_t* split_flags = nullptr,
            size_t max_rows_in_use = 0) {
    Ff2Args a;
    memset(&a, 0, sizeof(a));
    a.row_dst = row_dst;
    // K split across CTAs (small token tiles): needs the caller's scratch and zeroed flags; XMOE_FF2_SPLITK=0 turns it off
    static const bool splitk_enabled = [] {
        const char* e = getenv("XMOE_FF2_SPLITK");
        return !(e && e[0] == '0');
    }();
    // The K-split kernel is chosen here, from an upper bound of the tile count (the counts themselves are on the
    // device): it can only pay when the tiles cannot fill two rounds of SMs. The kernel then looks at the real
    // tile list and cuts tiles only if whole tiles would leave SM-rounds idle.
    if (splitk_enabled && nt <= 64 && num_sms() <= kMaxSplitCtas && max_rows_in_use > 0) {
        const size_t live_max = max_rows_in_use < (size_t)e_tot ? max_rows_in_use : (size_t)e_tot;
        const size_t token_tiles_max = live_max + max_rows_in_use / (size_t)nt;  // sum over experts of ceil(count / nt)
        const size_t tiles_max = token_tiles_max * (size_t)((H + 127) / 128);
        if (tiles_max <= 2 * (size_t)num_sms()) {
            a.split_partial = split_partial;
            a.split_flags = split_flags;
        }
    }
    // 256-token tiles run on CTA pairs (2-SM MMA) unless XMOE_FF2_PAIR=0: each CTA stages 128 token
    // rows and K 128 (64-byte weight rows). The single-CTA 256 variant uses K 64 (32-byte rows).
    static const bool pair_enabled = [] {
        const char* e = getenv("XMOE_FF2_PAIR");
        return !(e && e[0] == '0');
    }();
    const bool pair = nt >= 256 && pair_enabled && num_sms() >= 2 && H > 128 && I % 64 == 0;
    const bool k64 = nt >= 256 && !pair;
    // weight box: 128 rows x (small token tiles: 128 bytes = two K units; else 64 or 32 bytes)
    const bool wide = nt <= 64;
    int rc = make_tmap_2d(&a.tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w2_q, (uint64_t)I / 2, (uint64_t)e_tot * H,
                          wide ? 128 : (k64 ? 32 : 64), 128,
                          wide ? CU_TENSOR_MAP_SWIZZLE_128B
                               : (k64 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_64B));
    if (rc) return rc;
    a.tok3d = ((nt <= 64 && I % 64 == 0) || pair) ? 1 : 0;
    if (pair) {
        // one copy per K unit (two slabs of K 64) of the 128, 64 or 32 token rows a CTA stages
        if ((rc = make_tmap_kslabs(&a.tm_y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, yact, (uint64_t)I, rows, 128, 2)) ||
            (rc = make_tmap_kslabs(&a.tm_y_small, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, yact, (uint64_t)I, rows, 32, 2)) ||
            (rc = make_tmap_kslabs(&a.tm_y_mid, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, yact, (uint64_t)I, rows, 64, 2)))
            return rc;
    } else if (a.tok3d) {
        // small token tiles: one copy per two K units (K 256 = four slabs), for the full tile and for 8 / 16 rows
        if ((rc = make_tmap_kslabs(&a.tm_y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, yact, (uint64_t)I, rows, (uint32_t)nt, 4)) ||
            (rc = make_tmap_kslabs(&a.tm_y_small, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, yact, (uint64_t)I, rows, 8, 4)) ||
            (rc = make_tmap_kslabs(&a.tm_y_mid, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, yact, (uint64_t)I, rows, 16, 4)))
            return rc;
    } else {
        rc = make_tmap_2d(&a.tm_y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, yact, (uint64_t)I, rows, 64,
                          (uint32_t)(pair ? 128 : nt), CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
    }
    if (nt <= 64 && !a.tok3d) {
        rc = make_tmap_2d(&a.tm_y_small, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, yact, (uint64_t)I, rows, 64, 8,
                          CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
        rc = make_tmap_2d(&a.tm_y_mid, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, yact, (uint64_t)I, rows, 64, 16,
                          CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
    }
    a.scale2d = 0;
    if (nt <= 64 && H >= 128) {
        if ((rc = make_tmap_2d(&a.tm_s, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w2_scale, (uint64_t)H,
                               (uint64_t)e_tot * (uint64_t)((I + 127) / 128), 128, 2, CU_TENSOR_MAP_SWIZZLE_NONE)))
            return rc;
        a.scale2d = 1;
    }
    a.w2_scale = w2_scale;
    a.counts = counts;
    a.offsets = offsets;
    a.out = out_rows;
    a.status = status;
    a.E_tot = e_tot;
    a.H = H;
    a.I = I;
    a.groups = (I + 127) / 128;
    a.nt = nt;
    a.num_sms = num_sms();
    return pair ? launch_ff2_pair(a, stream) : launch_ff2(a, stream);
}

int forward_impl(const xmoe_config* cfg, const xmoe_weights* w, const void* x, const void* logits,
                 const int32_t* ext_idx, const void* ext_w, const float* ext_scale, int n, void* y, void* ws,
                 size_t ws_bytes, cudaStream_t stream, const int32_t* n_valid_dev = nullptr,
                 const xmoe_ep_buffers* ep_ret = nullptr, unsigned long long* row_dst = nullptr,
                 bool prequantised = false, bool scalars_precleared = false, void* scatter_rows = nullptr) {
    int rc = check_cfg(cfg);
    if (prequantised && (!ext_idx || !ext_scale || cfg->top_k + cfg->num_shared_experts != 1)) return XMOE_ERR_ARG;
    if (ep_ret && (!row_dst || !ext_idx || cfg->top_k + cfg->num_shared_experts != 1)) return XMOE_ERR_ARG;
    if (scatter_rows && (ep_ret || y)) return XMOE_ERR_ARG;
    if (rc) return rc;
    if (n < 0) return XMOE_ERR_ARG;
    if (n == 0) return XMOE_OK;
    if (n > (1 << 22)) return XMOE_ERR_LIMIT;
    if (!w || !x || !ws || (!logits && !ext_idx)) return XMOE_ERR_ARG;
    if (!y && !ext_idx && !scatter_rows) return XMOE_ERR_ARG;  // y may be null only when the rows stay in the workspace or go to scatter_rows
    if (!w->w13_packed || !w->w13_sf || !w->w13_gs || !w->w2_q || !w->w2_scale) return XMOE_ERR_ARG;
    if (reinterpret_cast<uintptr_t>(ws) & 1023u) return XMOE_ERR_WORKSPACE;
    const Layout L = make_layout(cfg, n);
    if (ws_bytes < L.total) return XMOE_ERR_WORKSPACE;
    uint8_t* b = (uint8_t*)ws;
    uint32_t* status = (uint32_t*)(b + L.off_status);
    uint32_t* amax_scratch = (uint32_t*)(b + L.off_amax);
    ActScale* scale = (ActScale*)(b + L.off_scale);
    int32_t* topk_idx = (int32_t*)(b + L.off_topk_idx);
    void* topk_w = b + L.off_topk_w;
    int32_t* topk_off = (int32_t*)(b + L.off_topk_off);
    int32_t* topk_row = (int32_t*)(b + L.off_topk_row);
    int32_t* counts = (int32_t*)(b + L.off_counts);
    int32_t* offsets = (int32_t*)(b + L.off_offsets);
    const int H = cfg->hidden, I = cfg->inter, E = cfg->num_experts;

    // status words (layer and gate), amax scratch, activation scale
    if (!scalars_precleared && cudaMemsetAsync(b, 0, kClearedBytes, stream) != cudaSuccess) return XMOE_ERR_CUDA;
    prof_mark(0, stream);

    // fork: the amax of x overlaps routing (joined before the quantiser)
    AmaxArgs am;
    am.x = x;
    am.n_elems = (size_t)n * H;
    am.scratch = amax_scratch;
    am.scale = scale;
    // worth it only when the pass is long enough to hide: at decode sizes the cross-stream edges cost
    // more than the few microseconds of amax
    const bool fork_pays = (size_t)n * H >= ((size_t)1 << 22);
    // tiny batches: every block of the quantiser takes the amax of x itself (one launch fewer)
    const bool fuse_amax = !ext_scale && !prequantised && (size_t)n * H <= ((size_t)1 << 18);
    SideStream* side = (ext_scale || prequantised || !fork_pays) ? nullptr : side_stream(stream);
    // Once the side stream has been forked off it is joined again on every way out of this function, error
    // returns included: a caller that is capturing `stream` into a graph must not be left with an unjoined fork.
    struct JoinOnExit {
        SideStream* side = nullptr;
        cudaStream_t caller = nullptr;
        void join() {
            if (!side) return;
            cudaEventRecord(side->join, side->stream);
            cudaStreamWaitEvent(caller, side->join, 0);
            side = nullptr;
        }
        ~JoinOnExit() { join(); }
    } forked;
    if (side) {
        if (cudaEventRecord(side->fork, stream) != cudaSuccess ||
            cudaStreamWaitEvent(side->stream, side->fork, 0) != cudaSuccess)
            return XMOE_ERR_CUDA;
        forked.side = side;
        forked.caller = stream;
        if ((rc = launch_act_amax(am, side->stream))) return rc;
        if (cudaEventRecord(side->join, side->stream) != cudaSuccess) return XMOE_ERR_CUDA;
    }

    // decode-sized batches with router-made routing: amax, router, permutation and quantiser are ONE launch
    static const bool front_enabled = [] { const char* e = getenv("XMOE_DECODE_FRONT"); return !(e && e[0] == '0'); }();
    // (measured, CUDA-graph replay of the layer at 16 tokens: Mixtral shape 178.7 -> 176.6 us, 1 token 73.1 -> 69.1,
    // Qwen3 47.2 -> 44.7, gpt-oss 172.3 -> 169.4; group-limited routing repeated in every CTA costs more than the
    // launches it saves, DeepSeek-V3 shape 510 -> 515 us, so that mode keeps the separate kernels)
    const bool grouped_routing = cfg->n_group > 1 || w->router_bias != nullptr;
    const bool use_front = front_enabled && logits && !ext_idx && !ext_scale && !prequantised && !n_valid_dev && fuse_amax &&
                           !grouped_routing && decode_front_applies(n, E, cfg->top_k, cfg->num_shared_experts, H);
    if (use_front) {
        FrontArgs f;
        f.x = x;
        f.logits = logits;
        f.expert_scale = w->expert_scale;
        f.scale = scale;
        f.topk_idx = topk_idx;
        f.topk_w = (uint16_t*)topk_w;
        f.topk_off = topk_off;
        f.topk_row = topk_row;
        f.counts = counts;
        f.offsets = offsets;
        f.row_token = (int32_t*)(b + L.off_row_token);
        f.row_weight = (uint16_t*)(b + L.off_row_weight);
        f.xq = b + L.off_xq;
        f.sfx = b + L.off_sfx;
        f.N = n;
        f.E = E;
        f.topk = cfg->top_k;
        f.n_shared = cfg->num_shared_experts;
        f.H = H;
        f.kb_pad = L.kb_pad;
        f.nt = L.nt;
        f.scoring = cfg->scoring;
        f.renorm = cfg->renormalize;
        f.routed_scale = cfg->routed_scale;
        if ((rc = launch_decode_front(f, stream))) return rc;
    } else if (ext_idx && (const void*)ext_idx == (const void*)topk_idx) {
        // routed in place: the gate GEMM of xmoe_forward_gated wrote the workspace's own arrays
    } else if (ext_idx) {
        // caller-supplied routing: widen [N, top_k] to the [N, k_eff] workspace arrays
        if (L.k_eff == cfg->top_k) {  // same row pitch: one flat copy each (a pitched copy of 4-byte rows is slow)
            if (cudaMemcpyAsync(topk_idx, ext_idx, (size_t)n * L.k_eff * 4, cudaMemcpyDeviceToDevice, stream) !=
                    cudaSuccess ||
                cudaMemcpyAsync(topk_w, ext_w, (size_t)n * L.k_eff * 2, cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
                return XMOE_ERR_CUDA;
        } else if (cudaMemcpy2DAsync(topk_idx, (size_t)L.k_eff * 4, ext_idx, (size_t)cfg->top_k * 4, (size_t)cfg->top_k * 4, n,
                              cudaMemcpyDeviceToDevice, stream) != cudaSuccess ||
            cudaMemcpy2DAsync(topk_w, (size_t)L.k_eff * 2, ext_w, (size_t)cfg->top_k * 2, (size_t)cfg->top_k * 2, n,
                              cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
            return XMOE_ERR_CUDA;
    } else {
        RouterArgs r;
        r.logits = logits;
        r.lut = w->sigmoid_lut;
        r.bias = w->router_bias;
        r.expert_scale = w->expert_scale;
        r.topk_idx = topk_idx;
        r.topk_w = topk_w;
        r.N = n;
        r.E = E;
        r.topk = cfg->top_k;
        r.idx_stride = L.k_eff;
        r.scoring = cfg->scoring;
        r.renorm = cfg->renormalize;
        r.n_group = cfg->n_group > 0 ? cfg->n_group : 1;
        r.topk_group = cfg->topk_group;
        r.routed_scale = cfg->routed_scale;
        if ((rc = launch_router_topk(r, stream))) return rc;
    }

    PackArgs p;
    p.topk_idx = topk_idx;
    p.topk_w = topk_w;
    p.N = n;
    p.E = E;
    p.topk = cfg->top_k;
    p.idx_stride = L.k_eff;
    p.n_shared = cfg->num_shared_experts;
    p.chunk_hist = (int32_t*)(b + L.off_hist);
    p.counts = counts;
    p.offsets = offsets;
    p.topk_off = topk_off;
    p.topk_row = topk_row;
    p.row_token = (int32_t*)(b + L.off_row_token);
    p.row_weight = b + L.off_row_weight;
    p.status = status;
    p.n_valid = n_valid_dev;
    prof_mark(1, stream);
    if (!use_front && (rc = launch_route_pack(p, stream))) return rc;
    if (ep_ret) {  // expert-parallel receive side: FF2 will store every row at its home rank
        if (cudaMemsetAsync(row_dst, 0, L.rows * 8, stream) != cudaSuccess) return XMOE_ERR_CUDA;
        if ((rc = launch_ep_row_dst(ep_ret, topk_row, row_dst, stream))) return rc;
    } else if (scatter_rows) {  // FF2 stores row (token, slot) at scatter_rows[token * k_eff + slot]
        row_dst = (unsigned long long*)(b + L.off_row_dst);
        if (cudaMemsetAsync(row_dst, 0, L.rows * 8, stream) != cudaSuccess) return XMOE_ERR_CUDA;
        if ((rc = launch_scatter_row_dst(topk_row, n * L.k_eff, H, scatter_rows, row_dst, stream))) return rc;
    }
    prof_mark(2, stream);

    if (ext_scale) {
        if (cudaMemcpyAsync(scale, ext_scale, 12, cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
            return XMOE_ERR_CUDA;
    } else if (side) {
        forked.side = nullptr;  // joined here
        if (cudaStreamWaitEvent(stream, side->join, 0) != cudaSuccess) return XMOE_ERR_CUDA;
    } else if (!prequantised && !fuse_amax && (rc = launch_act_amax(am, stream))) {
        return rc;
    }
    prof_mark(3, stream);

    QuantArgs q;
    q.x = x;
    q.scale = scale;
    q.topk_row = topk_row;
    q.N = n;
    q.H = H;
    q.k_eff = L.k_eff;
    q.idx_stride = L.k_eff;
    q.xq = b + L.off_xq;
    q.sfx = b + L.off_sfx;
    q.kb_pad = L.kb_pad;
    q.nt = L.nt;
    q.n_valid = n_valid_dev;
    q.fused_amax = fuse_amax;
    if (use_front) {
        // the packets are already there
    } else if (prequantised) {
        // x holds NVFP4 packets written by the sending ranks: codes [n, H/2], then block scales [n, H/16]
        if ((rc = launch_act_repack(x, (const uint8_t*)x + (size_t)n * (H / 2), q, stream))) return rc;
    } else if ((rc = launch_act_quant(q, stream))) {
        return rc;
    }
    prof_mark(4, stream);

    if ((rc = run_ff1(w->w13_packed, w->w13_sf, w->w13_gs, b + L.off_xq, b + L.off_sfx, (const float*)scale, counts,
                      offsets, b + L.off_row_weight, b + L.off_yact, status, L.e_tot, H, I, L.rows, L.nt,
                      cfg->activation, cfg->swiglu_alpha, cfg->swiglu_limit, stream)))
        return rc;
    prof_mark(5, stream);

    if (cfg->act_topk_keep > 0 && cfg->act_topk_keep < I) {
        ActTopkArgs t;
        t.yact = b + L.off_yact;
        t.counts = counts;
        t.offsets = offsets;
        t.E_tot = L.e_tot;
        t.I = I;
        t.keep = cfg->act_topk_keep;
        t.max_rows = (int)L.rows;
        if ((rc = launch_act_topk(t, stream))) return rc;
    }
    prof_mark(6, stream);

    if ((rc = run_ff2(w->w2_q, w->w2_scale, b + L.off_yact, counts, offsets, b + L.off_out, status, L.e_tot, H, I,
                      L.rows, ff2_token_tile(cfg, L.nt, (size_t)n * L.k_eff), stream,
                      (ep_ret || scatter_rows) ? row_dst : nullptr,
                      (float*)(b + L.off_ff2_partial), (uint32_t*)(b + kFf2FlagsOffset), (size_t)n * L.k_eff)))
        return rc;
    if (ep_ret && (rc = launch_ep_signal_ret(ep_ret, stream))) return rc;
    prof_mark(7, stream);

    CombineArgs c;
    c.rows = b + L.off_out;
    c.topk_row = topk_row;
    c.y = y;
    c.N = n;
    c.H = H;
    c.k_eff = L.k_eff;
    c.idx_stride = L.k_eff;
    rc = y ? launch_combine(c, stream) : XMOE_OK;
    prof_mark(8, stream);
    if (g_prof.ev && g_prof.step < g_prof.max_steps) ++g_prof.step;
    return rc;
}

}  // namespace

extern "C" {

const char* xmoe_build_info(void) {
    return "xmoe_b200 fused MoE: sm_100a, tcgen05 NVFP4 W4A4 FF1 + W4A16 FF2, CUDA " XMOE_STR(CUDART_VERSION);
}

const char* xmoe_status_string(int s) {
    switch (s) {
        case XMOE_OK: return "ok";
        case XMOE_ERR_ARG: return "bad argument (null pointer or non-positive size)";
        case XMOE_ERR_SHAPE: return "unsupported shape or configuration";
        case XMOE_ERR_WORKSPACE: return "workspace too small or not 1024-byte aligned";
        case XMOE_ERR_CUDA: return "CUDA runtime/driver call failed";
        case XMOE_ERR_TIMEOUT: return "a bounded device-side wait gave up";
        case XMOE_ERR_LIMIT: return "size beyond the supported maximum (for the *_static entry points: the fixed scratch array)";
        default: return "unknown status";
    }
}

size_t xmoe_packed_rows(const xmoe_config* cfg, int32_t n) {
    if (check_cfg(cfg) || n < 0) return 0;
    return packed_rows(cfg, n);
}
size_t xmoe_workspace_bytes(const xmoe_config* cfg, int32_t n) {
    if (check_cfg(cfg) || n < 0) return 0;
    return make_layout(cfg, n).total;
}
size_t xmoe_workspace_bytes_host_io(const xmoe_config* cfg, int32_t n) {
    if (check_cfg(cfg) || n < 0) return 0;
    return make_layout(cfg, n).total_host_io;
}

int xmoe_forward(const xmoe_config* cfg, const xmoe_weights* w, const void* x, const void* router_logits, int32_t n,
                 void* y, void* workspace, size_t workspace_bytes, xmoe_stream_t stream) {
    return forward_impl(cfg, w, x, router_logits, nullptr, nullptr, nullptr, n, y, workspace, workspace_bytes,
                        (cudaStream_t)stream);
}

int xmoe_forward_routed(const xmoe_config* cfg, const xmoe_weights* w, const void* x, const int32_t* topk_idx,
                        const void* topk_w, const float* act_scale, int32_t n, void* y, void* workspace,
                        size_t workspace_bytes, xmoe_stream_t stream) {
    if (!topk_idx || !topk_w) return XMOE_ERR_ARG;
    return forward_impl(cfg, w, x, nullptr, topk_idx, topk_w, act_scale, n, y, workspace, workspace_bytes,
                        (cudaStream_t)stream);
}

int xmoe_forward_routed_bounded(const xmoe_config* cfg, const xmoe_weights* w, const void* x, const int32_t* topk_idx,
                                const void* topk_w, const float* act_scale, int32_t n, const int32_t* n_valid_dev, void* y,
                                void* workspace, size_t workspace_bytes, xmoe_stream_t stream) {
    if (!topk_idx || !topk_w) return XMOE_ERR_ARG;
    return forward_impl(cfg, w, x, nullptr, topk_idx, topk_w, act_scale, n, y, workspace, workspace_bytes,
                        (cudaStream_t)stream, n_valid_dev);
}

int xmoe_forward_scatter(const xmoe_config* cfg, const xmoe_weights* w, const void* x, const void* router_logits,
                         const int32_t* topk_idx, const void* topk_w, const float* act_scale, int32_t n, void* rows_out,
                         void* workspace, size_t workspace_bytes, xmoe_stream_t stream) {
    if (!rows_out || (!router_logits && (!topk_idx || !topk_w))) return XMOE_ERR_ARG;
    return forward_impl(cfg, w, x, topk_idx ? nullptr : router_logits, topk_idx, topk_w, act_scale, n, nullptr, workspace,
                        workspace_bytes, (cudaStream_t)stream, nullptr, nullptr, nullptr, false, false, rows_out);
}

namespace {
// tensor maps of the gate GEMM: x [n, H] in boxes of min(n, 128) rows, gate_w [E, H] in one box of E rows
int gate_tmaps(const void* x, const void* gate_w, int n, int H, int E, CUtensorMap* tm_x, CUtensorMap* tm_w, int* n_pad,
               int* x_box, int* w_box) {
    if (H <= 0 || H % 64 || E <= 0 || E > 256) return XMOE_ERR_SHAPE;
    *n_pad = (E + 15) & ~15;
    *x_box = n < 128 ? n : 128;
    *w_box = E < *n_pad ? E : *n_pad;
    int rc = make_tmap_2d(tm_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, (uint64_t)H, (uint64_t)n, 64, (uint32_t)*x_box,
                          CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    return make_tmap_2d(tm_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, gate_w, (uint64_t)H, (uint64_t)E, 64, (uint32_t)*w_box,
                        CU_TENSOR_MAP_SWIZZLE_128B);
}
}  // namespace

int xmoe_gate_logits(const void* x, const void* gate_w, int32_t n, int32_t H, int32_t E, void* logits, uint32_t* status,
                     xmoe_stream_t stream) {
    if (!x || !gate_w || !logits || !status || n < 0) return XMOE_ERR_ARG;
    if (H <= 0 || H % 64 || E <= 0 || E > 256) return XMOE_ERR_SHAPE;
    if (n == 0) return XMOE_OK;
    CUtensorMap tm_x, tm_w;
    int n_pad, x_box, w_box;
    const int rc = gate_tmaps(x, gate_w, n, H, E, &tm_x, &tm_w, &n_pad, &x_box, &w_box);
    if (rc) return rc;
    return launch_gate_logits(tm_x, tm_w, logits, n, E, H, n_pad, x_box, w_box, status, (cudaStream_t)stream);
}

int xmoe_forward_gated(const xmoe_config* cfg, const xmoe_weights* w, const void* x, const void* gate_w,
                       void* logits_out, int32_t n, void* y, void* workspace, size_t workspace_bytes,
                       xmoe_stream_t stream) {
    if (!cfg || !w || !x || !gate_w || !workspace) return XMOE_ERR_ARG;
    int rc = check_cfg(cfg);
    if (rc) return rc;
    if (n < 0) return XMOE_ERR_ARG;
    if (n == 0) return XMOE_OK;
    if (n > (1 << 22)) return XMOE_ERR_LIMIT;
    if (reinterpret_cast<uintptr_t>(workspace) & 1023u) return XMOE_ERR_WORKSPACE;
    const Layout L = make_layout(cfg, n);
    if (workspace_bytes < L.total) return XMOE_ERR_WORKSPACE;
    uint8_t* b = (uint8_t*)workspace;
    uint32_t* gate_status = (uint32_t*)workspace + kGateStatusWord;
    CUtensorMap tm_x, tm_w;
    int n_pad, x_box, w_box;
    if ((rc = gate_tmaps(x, gate_w, n, cfg->hidden, cfg->num_experts, &tm_x, &tm_w, &n_pad, &x_box, &w_box))) return rc;
    if (cudaMemsetAsync(workspace, 0, kClearedBytes, (cudaStream_t)stream) != cudaSuccess) return XMOE_ERR_CUDA;
    // ONE kernel: gate GEMM, bf16 rounding of the logits, top-k and gate weights into the workspace's routing arrays
    RouterArgs r;
    r.logits = nullptr;
    r.lut = w->sigmoid_lut;
    r.bias = w->router_bias;
    r.expert_scale = w->expert_scale;
    r.topk_idx = (int32_t*)(b + L.off_topk_idx);
    r.topk_w = b + L.off_topk_w;
    r.N = n;
    r.E = cfg->num_experts;
    r.topk = cfg->top_k;
    r.idx_stride = L.k_eff;
    r.scoring = cfg->scoring;
    r.renorm = cfg->renormalize;
    r.n_group = cfg->n_group > 0 ? cfg->n_group : 1;
    r.topk_group = cfg->topk_group;
    r.routed_scale = cfg->routed_scale;
    if ((rc = launch_gate_route(tm_x, tm_w, logits_out, n, cfg->num_experts, cfg->hidden, n_pad, x_box, w_box, gate_status,
                                r, (cudaStream_t)stream)))
        return rc;
    // the layer takes the routing where it already lies (forward_impl recognises its own arrays)
    return forward_impl(cfg, w, x, nullptr, r.topk_idx, r.topk_w, nullptr, n, y, workspace, workspace_bytes,
                        (cudaStream_t)stream, nullptr, nullptr, nullptr, false, /*scalars_precleared=*/true);
}

int xmoe_probe_mma_rate(int32_t kind, int32_t n_mma, double* tflops_out, xmoe_stream_t stream) {
    return probe_mma_rate(kind, n_mma, tflops_out, (cudaStream_t)stream);
}

int xmoe_profile_begin(int32_t max_steps) {
    if (g_prof.ev) {
        for (size_t i = 0; i < (size_t)g_prof.max_steps * (kProfStages + 1); ++i) cudaEventDestroy(g_prof.ev[i]);
        delete[] g_prof.ev;
        g_prof = Profiler();
    }
    if (max_steps <= 0) return XMOE_OK;
    if (max_steps > 4096) return XMOE_ERR_LIMIT;
    const size_t n = (size_t)max_steps * (kProfStages + 1);
    g_prof.ev = new cudaEvent_t[n];
    for (size_t i = 0; i < n; ++i)
        if (cudaEventCreate(&g_prof.ev[i]) != cudaSuccess) return XMOE_ERR_CUDA;
    g_prof.max_steps = max_steps;
    g_prof.step = 0;
    return XMOE_OK;
}

int xmoe_profile_read(float* stage_ms_sum, int32_t* steps_out) {
    if (!stage_ms_sum || !steps_out) return XMOE_ERR_ARG;
    for (int i = 0; i < kProfStages; ++i) stage_ms_sum[i] = 0.f;
    *steps_out = g_prof.step;
    if (!g_prof.ev) return XMOE_OK;
    if (cudaDeviceSynchronize() != cudaSuccess) return XMOE_ERR_CUDA;
    for (int s = 0; s < g_prof.step; ++s) {
        cudaEvent_t* e = g_prof.ev + (size_t)s * (kProfStages + 1);
        for (int i = 0; i < kProfStages; ++i) {
            float ms = 0.f;
            if (cudaEventElapsedTime(&ms, e[i], e[i + 1]) != cudaSuccess) return XMOE_ERR_CUDA;
            stage_ms_sum[i] += ms;
        }
    }
    g_prof.step = 0;
    return XMOE_OK;
}

namespace {
int forward_host_impl(const xmoe_config* cfg, const xmoe_weights* w, const void* x_host, const void* logits_host,
                      int32_t n, void* y_host, void* workspace, size_t workspace_bytes, xmoe_stream_t stream, bool sync);
}

int xmoe_forward_host(const xmoe_config* cfg, const xmoe_weights* w, const void* x_host, const void* logits_host,
                      int32_t n, void* y_host, void* workspace, size_t workspace_bytes, xmoe_stream_t stream) {
    return forward_host_impl(cfg, w, x_host, logits_host, n, y_host, workspace, workspace_bytes, stream, true);
}

int xmoe_forward_host_async(const xmoe_config* cfg, const xmoe_weights* w, const void* x_host, const void* logits_host,
                            int32_t n, void* y_host, void* workspace, size_t workspace_bytes, xmoe_stream_t stream) {
    return forward_host_impl(cfg, w, x_host, logits_host, n, y_host, workspace, workspace_bytes, stream, false);
}

namespace {
int forward_host_impl(const xmoe_config* cfg, const xmoe_weights* w, const void* x_host, const void* logits_host,
                      int32_t n, void* y_host, void* workspace, size_t workspace_bytes, xmoe_stream_t stream, bool sync) {
    int rc = check_cfg(cfg);
    if (rc) return rc;
    if (n < 0 || !x_host || !logits_host || !y_host || !workspace) return XMOE_ERR_ARG;
    if (n == 0) return XMOE_OK;
    const Layout L = make_layout(cfg, n);
    if (workspace_bytes < L.total_host_io) return XMOE_ERR_WORKSPACE;
    cudaStream_t s = (cudaStream_t)stream;
    uint8_t* b = (uint8_t*)workspace;
    const size_t xb = (size_t)n * cfg->hidden * 2, lb = (size_t)n * cfg->num_experts * 2;
    if (cudaMemcpyAsync(b + L.off_x_in, x_host, xb, cudaMemcpyHostToDevice, s) != cudaSuccess ||
        cudaMemcpyAsync(b + L.off_logits_in, logits_host, lb, cudaMemcpyHostToDevice, s) != cudaSuccess)
        return XMOE_ERR_CUDA;
    rc = forward_impl(cfg, w, b + L.off_x_in, b + L.off_logits_in, nullptr, nullptr, nullptr, n, b + L.off_y_out,
                      workspace, workspace_bytes, s);
    if (rc) return rc;
    if (cudaMemcpyAsync(y_host, b + L.off_y_out, xb, cudaMemcpyDeviceToHost, s) != cudaSuccess) return XMOE_ERR_CUDA;
    if (sync && cudaStreamSynchronize(s) != cudaSuccess) return XMOE_ERR_CUDA;
    return XMOE_OK;
}
}  // namespace

int xmoe_read_status(const void* workspace, uint32_t* host_out, xmoe_stream_t stream) {
    if (!workspace || !host_out) return XMOE_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    // word 0: the layer's kernels; word kGateStatusWord: the gate GEMM of xmoe_forward_gated (the layer clears
    // only its own word, so a gate failure stays visible)
    uint32_t words[kGateStatusWord + 1];
    if (cudaMemcpyAsync(words, workspace, sizeof(words), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess)
        return XMOE_ERR_CUDA;
    *host_out = words[0] ? words[0] : words[kGateStatusWord];
    if (*host_out >= 0x100u && *host_out < 0x600u) return XMOE_ERR_TIMEOUT;
    return XMOE_OK;
}

int xmoe_workspace_view_get(const xmoe_config* cfg, int32_t n, void* workspace, size_t workspace_bytes,
                            xmoe_workspace_view* v) {
    int rc = check_cfg(cfg);
    if (rc) return rc;
    if (!workspace || !v || n <= 0) return XMOE_ERR_ARG;
    const Layout L = make_layout(cfg, n);
    if (workspace_bytes < L.total) return XMOE_ERR_WORKSPACE;
    uint8_t* b = (uint8_t*)workspace;
    v->status = (uint32_t*)(b + L.off_status);
    v->act_scale = (float*)(b + L.off_scale);
    v->topk_idx = (int32_t*)(b + L.off_topk_idx);
    v->topk_w = b + L.off_topk_w;
    v->topk_off = (int32_t*)(b + L.off_topk_off);
    v->topk_row = (int32_t*)(b + L.off_topk_row);
    v->counts = (int32_t*)(b + L.off_counts);
    v->offsets = (int32_t*)(b + L.off_offsets);
    v->row_token = (int32_t*)(b + L.off_row_token);
    v->row_weight = b + L.off_row_weight;
    v->xq = b + L.off_xq;
    v->sfx = b + L.off_sfx;
    v->yact = b + L.off_yact;
    v->out_rows = b + L.off_out;
    v->k_eff = L.k_eff;
    v->packed_rows = (int32_t)L.rows;
    v->kb_pad = L.kb_pad;
    v->token_tile = L.nt;
    return XMOE_OK;
}

int xmoe_router_topk(const void* router_logits, const float* router_bias, const float* sigmoid_lut,
                     const void* expert_scale, int32_t n, int32_t E, int32_t top_k, int32_t idx_stride, int32_t scoring,
                     int32_t renormalize, int32_t n_group, int32_t topk_group, float routed_scale, int32_t* topk_idx,
                     void* topk_w, xmoe_stream_t stream) {
    if (n < 0 || !router_logits || !topk_idx || !topk_w) return XMOE_ERR_ARG;
    if (E <= 0 || E > 1024 || top_k <= 0 || top_k > 8 || top_k > E || idx_stride < top_k) return XMOE_ERR_SHAPE;
    RouterArgs r;
    r.logits = router_logits;
    r.lut = sigmoid_lut;
    r.bias = router_bias;
    r.expert_scale = expert_scale;
    r.topk_idx = topk_idx;
    r.topk_w = topk_w;
    r.N = n;
    r.E = E;
    r.topk = top_k;
    r.idx_stride = idx_stride;
    r.scoring = scoring;
    r.renorm = renormalize;
    r.n_group = n_group > 0 ? n_group : 1;
    r.topk_group = topk_group;
    r.routed_scale = routed_scale;
    return launch_router_topk(r, (cudaStream_t)stream);
}

size_t xmoe_route_pack_scratch_bytes(int32_t n, int32_t E, int32_t n_shared) {
    return (size_t)route_pack_chunks(n > 0 ? n : 1) * (size_t)(E + n_shared) * 4;
}

int xmoe_route_pack(int32_t* topk_idx, void* topk_w, int32_t n, int32_t E, int32_t top_k, int32_t idx_stride,
                    int32_t n_shared, void* scratch, int32_t* counts, int32_t* offsets, int32_t* topk_off,
                    int32_t* topk_row, int32_t* row_token, void* row_weight, uint32_t* status, xmoe_stream_t stream) {
    if (n < 0 || !topk_idx || !topk_w || !scratch || !counts || !offsets || !topk_off || !topk_row || !row_token ||
        !row_weight || !status)
        return XMOE_ERR_ARG;
    if (idx_stride < top_k + n_shared) return XMOE_ERR_SHAPE;
    PackArgs p;
    p.topk_idx = topk_idx;
    p.topk_w = topk_w;
    p.N = n;
    p.E = E;
    p.topk = top_k;
    p.idx_stride = idx_stride;
    p.n_shared = n_shared;
    p.chunk_hist = (int32_t*)scratch;
    p.counts = counts;
    p.offsets = offsets;
    p.topk_off = topk_off;
    p.topk_row = topk_row;
    p.row_token = row_token;
    p.row_weight = row_weight;
    p.status = status;
    return launch_route_pack(p, (cudaStream_t)stream);
}

int32_t xmoe_route_pack_static_max_tokens(void) { return route_pack_static_max_tokens(); }

int xmoe_route_pack_static(int32_t* topk_idx, void* topk_w, int32_t n, int32_t E, int32_t top_k, int32_t idx_stride,
                           int32_t n_shared, int32_t* counts, int32_t* offsets, int32_t* topk_off, int32_t* topk_row,
                           int32_t* row_token, void* row_weight, uint32_t* status, xmoe_stream_t stream) {
    if (n < 0 || !topk_idx || !topk_w || !counts || !offsets || !topk_off || !topk_row || !row_token || !row_weight ||
        !status)
        return XMOE_ERR_ARG;
    if (idx_stride < top_k + n_shared) return XMOE_ERR_SHAPE;
    PackArgs p;
    p.topk_idx = topk_idx;
    p.topk_w = topk_w;
    p.N = n;
    p.E = E;
    p.topk = top_k;
    p.idx_stride = idx_stride;
    p.n_shared = n_shared;
    p.chunk_hist = nullptr;  // filled in with the library's own fixed device array
    p.counts = counts;
    p.offsets = offsets;
    p.topk_off = topk_off;
    p.topk_row = topk_row;
    p.row_token = row_token;
    p.row_weight = row_weight;
    p.status = status;
    return launch_route_pack_static(p, (cudaStream_t)stream);
}

int xmoe_act_amax(const void* x, size_t n_elems, uint32_t* scratch, float* act_scale, xmoe_stream_t stream) {
    if (!x || !scratch || !act_scale || !n_elems) return XMOE_ERR_ARG;
    AmaxArgs a;
    a.x = x;
    a.n_elems = n_elems;
    a.scratch = scratch;
    a.scale = (ActScale*)act_scale;
    return launch_act_amax(a, (cudaStream_t)stream);
}

int xmoe_act_scale_from_amax(const float* amax, float* act_scale, xmoe_stream_t stream) {
    if (!amax || !act_scale) return XMOE_ERR_ARG;
    return launch_act_scale_from_amax(amax, act_scale, (cudaStream_t)stream);
}

int xmoe_act_quant_pack(const void* x, const float* act_scale, const int32_t* topk_row, int32_t n, int32_t H,
                        int32_t k_eff, int32_t idx_stride, int32_t token_tile, void* xq, void* sfx,
                        xmoe_stream_t stream) {
    if (!x || !act_scale || !topk_row || !xq || !sfx || n < 0) return XMOE_ERR_ARG;
    if (H <= 0 || H % 64 || k_eff <= 0 || idx_stride < k_eff) return XMOE_ERR_SHAPE;
    QuantArgs q;
    q.x = x;
    q.scale = (const ActScale*)act_scale;
    q.topk_row = topk_row;
    q.N = n;
    q.H = H;
    q.k_eff = k_eff;
    q.idx_stride = idx_stride;
    q.xq = xq;
    q.sfx = sfx;
    q.kb_pad = (int)align_up((size_t)H / 64, 4);
    q.nt = token_tile;
    q.n_valid = nullptr;
    q.fused_amax = false;
    return launch_act_quant(q, (cudaStream_t)stream);
}

int xmoe_ff1(const void* w13_packed, const void* w13_sf, const float* w13_gs, const void* xq, const void* sfx,
             const float* act_scale, const int32_t* counts, const int32_t* offsets, const void* row_weight, void* yact,
             uint32_t* status, int32_t e_tot, int32_t H, int32_t I, int32_t packed_rows_, int32_t token_tile,
             int32_t activation, float alpha, float limit, xmoe_stream_t stream) {
    if (!w13_packed || !w13_sf || !w13_gs || !xq || !sfx || !act_scale || !counts || !offsets || !row_weight ||
        !yact || !status)
        return XMOE_ERR_ARG;
    if (e_tot <= 0 || H <= 0 || I <= 0 || packed_rows_ <= 0 || packed_rows_ % 128 || H % 64 || I % 32)
        return XMOE_ERR_SHAPE;
    return run_ff1(w13_packed, w13_sf, w13_gs, xq, sfx, act_scale, counts, offsets, row_weight, yact, status, e_tot, H,
                   I, (size_t)packed_rows_, token_tile, activation, alpha, limit, (cudaStream_t)stream);
}

int xmoe_act_topk(void* yact, const int32_t* counts, const int32_t* offsets, int32_t e_tot, int32_t I, int32_t keep,
                  int32_t packed_rows_, xmoe_stream_t stream) {
    if (!yact || !counts || !offsets) return XMOE_ERR_ARG;
    ActTopkArgs t;
    t.yact = yact;
    t.counts = counts;
    t.offsets = offsets;
    t.E_tot = e_tot;
    t.I = I;
    t.keep = keep;
    t.max_rows = packed_rows_;
    return launch_act_topk(t, (cudaStream_t)stream);
}

int xmoe_ff2(const void* w2_q, const void* w2_scale, const void* yact, const int32_t* counts, const int32_t* offsets,
             void* out_rows, uint32_t* status, int32_t e_tot, int32_t H, int32_t I, int32_t packed_rows_,
             int32_t token_tile, xmoe_stream_t stream) {
    if (!w2_q || !w2_scale || !yact || !counts || !offsets || !out_rows || !status) return XMOE_ERR_ARG;
    if (e_tot <= 0 || H <= 0 || I <= 0 || packed_rows_ <= 0 || packed_rows_ % 128 || H % 8 || I % 32)
        return XMOE_ERR_SHAPE;
    return run_ff2(w2_q, w2_scale, yact, counts, offsets, out_rows, status, e_tot, H, I, (size_t)packed_rows_,
                   token_tile, (cudaStream_t)stream);
}

int xmoe_ep_post_counts(const xmoe_ep_buffers* b, const int32_t* counts_global, const float* amax_local,
                        xmoe_stream_t stream) {
    return launch_ep_post_counts(b, counts_global, amax_local, (cudaStream_t)stream);
}
int xmoe_ep_dispatch(const xmoe_ep_buffers* b, const void* x, const int32_t* topk_idx, const void* topk_w,
                     const int32_t* topk_off, const int32_t* counts_global, int32_t n_tokens, int32_t top_k,
                     int32_t idx_stride, float* amax_global, xmoe_stream_t stream) {
    return launch_ep_dispatch(b, x, topk_idx, topk_w, topk_off, counts_global, n_tokens, top_k, idx_stride, amax_global,
                              (cudaStream_t)stream);
}
int xmoe_ep_wait_data(const xmoe_ep_buffers* b, int32_t* e_recv, void* w_recv, int32_t* n_recv, xmoe_stream_t stream) {
    return launch_ep_wait_data(b, e_recv, w_recv, n_recv, (cudaStream_t)stream);
}
int xmoe_ep_return(const xmoe_ep_buffers* b, const void* out_rows, const int32_t* topk_row, int32_t expected_rows,
                   xmoe_stream_t stream) {
    return launch_ep_return(b, out_rows, topk_row, expected_rows, (cudaStream_t)stream);
}
int xmoe_ep_forward_local(const xmoe_ep_buffers* b, const xmoe_config* cfg, const xmoe_weights* w,
                          const int32_t* e_recv, const void* w_recv, const float* act_scale, const int32_t* n_recv_dev,
                          int32_t quantised_input, void* row_dst_scratch, void* workspace, size_t workspace_bytes,
                          xmoe_stream_t stream) {
    if (!b || !e_recv || !w_recv || !row_dst_scratch || b->rank < 0 || b->rank >= XMOE_EP_MAX_WORLD) return XMOE_ERR_ARG;
    if (!cfg || cfg->hidden != b->hidden || cfg->num_experts != b->experts_per_rank) return XMOE_ERR_SHAPE;
    return forward_impl(cfg, w, b->recv_x[b->rank], nullptr, e_recv, w_recv, act_scale, b->cap_rows, nullptr, workspace,
                        workspace_bytes, (cudaStream_t)stream, n_recv_dev, b, (unsigned long long*)row_dst_scratch,
                        quantised_input != 0);
}
int xmoe_ep_dispatch_quantised(const xmoe_ep_buffers* b, const void* x, const int32_t* topk_idx, const void* topk_w,
                               const int32_t* topk_off, const int32_t* counts_global, int32_t n_tokens, int32_t top_k,
                               int32_t idx_stride, float* amax_global, xmoe_stream_t stream) {
    return launch_ep_dispatch_q(b, x, topk_idx, topk_w, topk_off, counts_global, n_tokens, top_k, idx_stride, amax_global,
                                (cudaStream_t)stream);
}
int xmoe_ep_wait_ret(const xmoe_ep_buffers* b, xmoe_stream_t stream) {
    return launch_ep_wait_ret(b, (cudaStream_t)stream);
}
int xmoe_ep_status(const xmoe_ep_buffers* b, xmoe_stream_t stream, uint32_t* bits_out) {
    if (!b || !bits_out || b->rank < 0 || b->rank >= XMOE_EP_MAX_WORLD || !b->ctl[b->rank]) return XMOE_ERR_ARG;
    if (cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess) return XMOE_ERR_CUDA;
    // the sticky error word sits after the count table, the amax slots, three flag arrays and three counters
    const size_t off = (64 + 8 + 24 + 3) * 4;
    if (cudaMemcpy(bits_out, (const uint8_t*)b->ctl[b->rank] + off, 4, cudaMemcpyDeviceToHost) != cudaSuccess)
        return XMOE_ERR_CUDA;
    return XMOE_OK;
}

int xmoe_combine(const void* out_rows, const int32_t* topk_row, int32_t n, int32_t H, int32_t k_eff, int32_t idx_stride,
                 void* y, xmoe_stream_t stream) {
    if (!out_rows || !topk_row || !y || n < 0) return XMOE_ERR_ARG;
    CombineArgs c;
    c.rows = out_rows;
    c.topk_row = topk_row;
    c.y = y;
    c.N = n;
    c.H = H;
    c.k_eff = k_eff;
    c.idx_stride = idx_stride;
    return launch_combine(c, (cudaStream_t)stream);
}

size_t xmoe_nvfp4_sf_bytes(int32_t n_mats, int32_t rows, int32_t k) {
    if (n_mats <= 0 || rows <= 0 || k <= 0) return 0;
    return (size_t)n_mats * ((rows + 127) / 128) * align_up((size_t)k / 64, 4) * 512;
}

int xmoe_prep_nvfp4_sf(const void* sf_in, void* sf_out, int32_t n_mats, int32_t rows, int32_t k, xmoe_stream_t stream) {
    if (!sf_in || !sf_out) return XMOE_ERR_ARG;
    if (n_mats <= 0 || rows <= 0 || k <= 0 || k % 64) return XMOE_ERR_SHAPE;
    return launch_prep_nvfp4_sf(sf_in, sf_out, n_mats, rows, k / 16, (rows + 127) / 128,
                                (int)align_up((size_t)k / 64, 4), (cudaStream_t)stream);
}

int xmoe_repack_gptq(const void* qweight, void* out, int32_t num_mats, int32_t k, int32_t o, xmoe_stream_t stream) {
    if (!qweight || !out) return XMOE_ERR_ARG;
    if (num_mats <= 0 || k <= 0 || o <= 0) return XMOE_ERR_SHAPE;
    return launch_repack_gptq(qweight, out, num_mats, k, o, (cudaStream_t)stream);
}

int xmoe_repack_int4_kmajor(const void* w_in, void* out, size_t n_words, xmoe_stream_t stream) {
    if (!w_in || !out) return XMOE_ERR_ARG;
    return launch_repack_kmajor_int4(w_in, out, n_words, (cudaStream_t)stream);
}

void xmoe_fill_sigmoid_lut(float* host_out) {
    if (!host_out) return;
    for (uint32_t i = 0; i < 65536u; ++i) {
        const uint32_t bits = i << 16;
        float x;
        memcpy(&x, &bits, 4);
        host_out[i] = (float)(1.0 / (1.0 + std::exp(-(double)x)));
    }
}

}  // extern "C"
