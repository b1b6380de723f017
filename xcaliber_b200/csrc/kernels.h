// Internal launcher interface between the C ABI (api.cu) and the kernel translation
// units. Plain structs of device pointers and sizes; every launcher enqueues on the
// given stream and returns an XMOE_* status without synchronising.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>

#include "../../include/xmoe_b200.h"

namespace xmoe {

// Function attributes, occupancy answers and SM counts belong to a DEVICE, not to the process: a host
// that drives several GPUs sets and caches them once per device. Caches are arrays indexed by this slot
// (-1: no current device or an ordinal beyond kMaxDevices, reported as XMOE_ERR_CUDA by the callers).
constexpr int kMaxDevices = 64;
inline int device_slot() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
    return dev;
}

struct RouterArgs {
    const void* logits;        // bf16 [N, E]
    const float* lut;          // fp32 [65536] sigmoid table (grouped mode only)
    const float* bias;         // fp32 [E] selection bias or null
    const void* expert_scale;  // bf16 [E] or null
    int32_t* topk_idx;         // [N, idx_stride]
    void* topk_w;              // bf16 [N, idx_stride]
    int N, E, topk, idx_stride;
    int scoring;               // 0 softmax, 1 sigmoid
    int renorm;
    int n_group, topk_group;
    float routed_scale;
};

struct PackArgs {
    int32_t* topk_idx;   // [N, idx_stride]; shared-expert slots are filled in here
    void* topk_w;        // bf16 [N, idx_stride]
    int N, E, topk, idx_stride, n_shared;
    int32_t* chunk_hist; // [chunks, E + n_shared]
    int32_t* counts;     // [E + n_shared]
    int32_t* offsets;    // [E + n_shared + 1], multiples of 128
    int32_t* topk_off;   // [N, idx_stride] rank inside the expert
    int32_t* topk_row;   // [N, idx_stride] absolute packed row
    int32_t* row_token;  // [R_cap]
    void* row_weight;    // bf16 [R_cap]
    uint32_t* status;
    const int32_t* n_valid = nullptr;  // optional, device: tokens at and beyond *n_valid are not in use and are not walked
};

struct ActScale {  // same meaning as the reference's MoeActScale (preamble.cuh:12-15)
    float xgs;      // 2688 / amax
    float xgs_inv;  // bf16(amax / 2688) widened to fp32
};

struct AmaxArgs {
    const void* x;  // bf16 [N, H]
    size_t n_elems;
    uint32_t* scratch;  // [2]: running max, ticket (both zero on entry, zero on exit)
    ActScale* scale;  // 4 floats of room: xgs, xgs_inv, amax, unused
};

struct QuantArgs {
    const void* x;  // bf16 [N, H]
    const ActScale* scale;
    const int32_t* topk_row;  // [N, idx_stride]
    int N, H, k_eff, idx_stride;
    void* xq;   // u8 [R_cap, H/2]
    void* sfx;  // u8 [R_cap/nt, KB, 512]
    int kb_pad; // K blocks of 64 per row, rounded up to a multiple of 4
    int nt;     // token tile the scale-factor tiles are laid out for: 32, 64 or 128
    const int32_t* n_valid;  // optional, device: tokens at and beyond *n_valid have no rows and are not scanned
    bool fused_amax;         // small batches: the kernel takes the amax of x itself and writes *scale (no amax kernel)
};

// The front of the layer in one launch for decode-sized batches (decode_front.cu): amax + scale, router, permutation,
// NVFP4 packets, for flat (softmax or sigmoid) routing. Fields as in RouterArgs / PackArgs / QuantArgs; idx_stride of
// the routing arrays = topk + n_shared.
struct FrontArgs {
    const void* x;             // bf16 [N, H]
    const void* logits;        // bf16 [N, E]
    const void* expert_scale;  // bf16 [E] or null
    ActScale* scale;           // out: {XGS, XGSINV, amax}
    int32_t* topk_idx;
    uint16_t* topk_w;
    int32_t* topk_off;
    int32_t* topk_row;
    int32_t* counts;
    int32_t* offsets;
    int32_t* row_token;
    uint16_t* row_weight;
    uint8_t* xq;
    uint8_t* sfx;
    int N, E, topk, n_shared, H, kb_pad, nt;
    int scoring, renorm;
    float routed_scale;
};

struct Ff1Args {
    CUtensorMap tm_w;  // u8 [E_tot*2I, H/2], box 128 B x 128 rows, 128-byte swizzle
    CUtensorMap tm_x;  // u8 [R_cap, H/2], box 128 B x NT rows
    const uint8_t* sfw;      // [E_tot, 2, MB, KB, 512]
    const uint8_t* sfx;      // [R_cap/nt, KB, 512]
    const float* w13_gs;     // [E_tot, 2]
    const ActScale* scale;
    const int32_t* counts;
    const int32_t* offsets;
    const void* row_weight;  // bf16 [R_cap]
    void* yact;              // bf16 [R_cap, I]
    uint32_t* status;
    int E_tot, H, I, kb_pad, mb;  // mb = ceil(I / 128)
    int nt;                       // token tile: 32, 64 or 128
    int activation;               // 0 silu*up, 1 clamped swiglu, 2 gelu_tanh*up
    float alpha, limit;
    int num_sms;
};

struct Ff2Args {
    CUtensorMap tm_w;  // u8 [E_tot*H, I/2], box (128 | 64 | 32) B x 128 rows, swizzle = box width
    CUtensorMap tm_y;  // bf16 [R_cap, I], box 64 elems x NT rows, 128-byte swizzle
    // The same tensor with smaller boxes, used when a tile holds few tokens. Token tiles of NT <= 64: 8 and
    // 16 rows (the MMA still reads NT rows; the columns of the stale ones are never stored). CTA pairs: 32 and
    // 64 rows per CTA (the MMA N is the tile's rows rounded up to 32, each CTA stages half of them).
    CUtensorMap tm_y_small, tm_y_mid;
    // tok3d (NT <= 64 with I % 64 == 0, and always on CTA pairs): the three maps above are 3-D views
    // [I/64][R_cap][64] of the same tensor with boxes of kblocks x rows x 64, so that ONE copy fetches K 256
    // (NT <= 64) or K 128 (pairs) of a token tile as 128-byte-swizzle slabs of K 64
    int tok3d;
    // NT <= 64 and H >= 128: the scales as a 2-D tensor [E_tot * G, H] with boxes of 2 groups x 128 features, so that
    // ONE copy fetches the scales of both K units of a weight stage (scale2d = 1)
    CUtensorMap tm_s;
    int scale2d;
    const void* w2_scale;  // bf16 [E_tot, G, H]
    const int32_t* counts;
    const int32_t* offsets;
    void* out;  // bf16 [R_cap, H]
    // optional [R_cap]: where each packed row's output goes instead of `out` (byte address of the row
    // start, 0 = nowhere). Expert-parallel ranks point it at the home ranks' return buffers, so that
    // the epilogue's stores are the return transfer.
    const unsigned long long* row_dst;
    uint32_t* status;
    // Tiles cut along K across CTAs (token tiles of NT <= 64 only; both null = whole tiles per CTA):
    // split_partial fp32 [CTAs][NT][128], one slot per CTA; split_flags u32 [CTAs], ZERO at launch.
    float* split_partial;
    uint32_t* split_flags;
    int E_tot, H, I, groups;  // groups = ceil(I / 128)
    int nt;
    int num_sms;
};

struct CombineArgs {
    const void* rows;         // bf16 [R_cap, H]
    const int32_t* topk_row;  // [N, idx_stride]
    void* y;                  // bf16 [N, H]
    int N, H, k_eff, idx_stride;
};

struct ActTopkArgs {
    void* yact;  // bf16 [R_cap, I], sparsified in place
    const int32_t* counts;
    const int32_t* offsets;
    int E_tot, I, keep;
    int max_rows;  // grid bound (R_cap)
};

int launch_router_topk(const RouterArgs& a, cudaStream_t stream);
int route_pack_chunks(int N);
int launch_route_pack(const PackArgs& a, cudaStream_t stream);
int route_pack_static_max_tokens();
int launch_route_pack_static(PackArgs a, cudaStream_t stream);  // scratch = a fixed device array of the library
int launch_act_amax(const AmaxArgs& a, cudaStream_t stream);
bool decode_front_applies(int N, int E, int topk, int n_shared, int H);
int launch_decode_front(const FrontArgs& a, cudaStream_t stream);
int launch_act_scale_from_amax(const float* amax, float* scale, cudaStream_t stream);
int launch_act_quant(const QuantArgs& a, cudaStream_t stream);
// rows already quantised by a peer: codes [N, H/2] + block scales [N, H/16] -> a.xq / a.sfx (a.x and a.scale unused)
int launch_act_repack(const void* xq_in, const void* sf_in, const QuantArgs& a, cudaStream_t stream);
int launch_ff1(const Ff1Args& a, cudaStream_t stream);
int launch_ff1_prefill(const Ff1Args& a, cudaStream_t stream);
int launch_ff1_pair(const Ff1Args& a, cudaStream_t stream);  // 256-token tiles on CTA pairs (2-SM MMA)
int launch_ff2(const Ff2Args& a, cudaStream_t stream);
int launch_ff2_pair(const Ff2Args& a, cudaStream_t stream);  // 256-token tiles on CTA pairs (2-SM MMA)
int launch_combine(const CombineArgs& a, cudaStream_t stream);
int launch_act_topk(const ActTopkArgs& a, cudaStream_t stream);
// topk_row is [N, k_eff] dense (n_slots = N * k_eff); row_dst must be zero on entry
int launch_scatter_row_dst(const int32_t* topk_row, int n_slots, int hidden, void* rows_out, unsigned long long* row_dst,
                           cudaStream_t stream);
int launch_prep_nvfp4_sf(const void* sf_in, void* sf_out, int n_mats, int rows, int kblocks16, int mb, int kb_pad,
                         cudaStream_t stream);
int launch_repack_gptq(const void* qweight, void* out, int E, int K, int O, cudaStream_t stream);
int launch_ep_post_counts(const xmoe_ep_buffers* b, const int32_t* counts_global, const float* amax_local,
                          cudaStream_t stream);
int launch_ep_dispatch(const xmoe_ep_buffers* b, const void* x, const int32_t* topk_idx, const void* topk_w,
                       const int32_t* topk_off, const int32_t* counts_global, int n, int top_k, int idx_stride,
                       float* amax_global, cudaStream_t stream);
int launch_ep_dispatch_q(const xmoe_ep_buffers* b, const void* x, const int32_t* topk_idx, const void* topk_w,
                         const int32_t* topk_off, const int32_t* counts_global, int n, int top_k, int idx_stride,
                         float* amax_global, cudaStream_t stream);
int launch_ep_wait_data(const xmoe_ep_buffers* b, int32_t* e_recv, void* w_recv, int32_t* n_recv, cudaStream_t stream);
int launch_ep_return(const xmoe_ep_buffers* b, const void* out_rows, const int32_t* topk_row, int expected_rows,
                     cudaStream_t stream);
int launch_ep_wait_ret(const xmoe_ep_buffers* b, cudaStream_t stream);
int launch_ep_row_dst(const xmoe_ep_buffers* b, const int32_t* topk_row, unsigned long long* row_dst, cudaStream_t stream);
int launch_ep_signal_ret(const xmoe_ep_buffers* b, cudaStream_t stream);
// tm_x: bf16 [n, H] box 64 x x_box_rows; tm_w: bf16 [E, H] box 64 x w_box_rows (rows beyond a box are
// stale shared memory and only feed accumulator rows / columns that are never stored)
int launch_gate_logits(const CUtensorMap& tm_x, const CUtensorMap& tm_w, void* logits, int n, int E, int H, int n_pad,
                       int x_box_rows, int w_box_rows, uint32_t* status, cudaStream_t stream);
int launch_gate_route(const CUtensorMap& tm_x, const CUtensorMap& tm_w, void* logits, int n, int E, int H, int n_pad,
                      int x_box_rows, int w_box_rows, uint32_t* status, const RouterArgs& r, cudaStream_t stream);
int probe_mma_rate(int kind, int n_mma, double* tflops_out, cudaStream_t stream);
int launch_repack_kmajor_int4(const void* w_in, void* out, size_t n_words, cudaStream_t stream);

}  // namespace xmoe
