/*
 * xmoe_b200.h -- C ABI of the B200 (sm_100a) fused Mixture-of-Experts layer.
 *
 * This is the drop-in boundary for the fused-MoE hot path of xCaliber. Each entry point
 * names the reference interface it replaces (paths are relative to the xCaliber tree).
 * All pointers are DEVICE pointers unless the name says host. Every function enqueues
 * on `stream` and returns immediately with one of the XMOE_* status codes below; none
 * of them allocates device memory (the caller owns the workspace) and none of them
 * synchronises, except xmoe_forward_host and xmoe_read_status.
 *
 * Tensor contracts (row-major, innermost dimension last):
 *   x               bf16 [N, H]                activations
 *   router_logits   bf16 [N, E]                gate output (the gate GEMM stays outside, as
 *                                              in the reference: method.py:240-264)
 *   w13_packed      u8   [E_tot, 2I, H/2]      NVFP4 E2M1 pairs, low nibble = lower K, rows
 *                                              [0,I) gate (W1) and [I,2I) up (W3): the
 *                                              checkpoint layout of xR64FF1.cu:17-20
 *   w13_sf          u8   prepared by xmoe_prep_nvfp4_sf from E4M3 [E_tot, 2I, H/16]
 *   w13_gs          f32  [E_tot, 2]            dequant multipliers (gate, up)
 *   w2_q            u32  [E_tot, H, I/8]       int4 (offset binary), prepared by
 *                                              xmoe_repack_gptq / xmoe_repack_int4_kmajor
 *   w2_scale        bf16 [E_tot, I/128, H]     group-128 scales (GPTQ order: group major)
 *   y               bf16 [N, H]
 * E_tot = num_experts + num_shared_experts; shared experts are the trailing matrices.
 */
#ifndef XMOE_B200_H_
#define XMOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define XMOE_OK 0
#define XMOE_ERR_ARG 1
#define XMOE_ERR_SHAPE 2
#define XMOE_ERR_WORKSPACE 3
#define XMOE_ERR_CUDA 4
#define XMOE_ERR_TIMEOUT 5
#define XMOE_ERR_LIMIT 6

typedef void* xmoe_stream_t; /* a cudaStream_t */

typedef struct xmoe_config {
    int32_t hidden;             /* H, multiple of 64 */
    int32_t inter;              /* I, multiple of 32 */
    int32_t num_experts;        /* E <= 1024 routed experts */
    int32_t top_k;              /* 1..8 */
    int32_t num_shared_experts; /* 0..8, every token, weight 1 */
    int32_t scoring;            /* 0 softmax, 1 sigmoid */
    int32_t renormalize;        /* normalise the k gate weights to sum 1 (reference: always) */
    int32_t n_group;            /* 1 = flat routing */
    int32_t topk_group;
    int32_t activation;         /* 0 silu(g)*u, 1 clamped swiglu (alpha, limit), 2 gelu_tanh(g)*u */
    int32_t act_topk_keep;      /* 0 = dense; else entries kept per FF1 output row */
    int32_t token_tile;         /* 0 = choose from N; else 32, 64 or 128 */
    float routed_scale;
    float swiglu_alpha;
    float swiglu_limit;
} xmoe_config;

typedef struct xmoe_weights {
    const void* w13_packed;
    const void* w13_sf;
    const float* w13_gs;
    const void* w2_q;
    const void* w2_scale;
    const float* router_bias;  /* f32 [E] selection bias, or NULL */
    const void* expert_scale;  /* bf16 [E] per-expert output scale, or NULL */
    const float* sigmoid_lut;  /* f32 [65536], required when n_group > 1 or router_bias != NULL */
} xmoe_weights;

/* ---- whole layer ------------------------------------------------------------------- */

/* Replaces _C.build_info (vllm/csrc/xr64_abs_bridge.cu:239-241). Static string. */
const char* xmoe_build_info(void);
const char* xmoe_status_string(int status);

/* Packed-row capacity and workspace size for a batch of N tokens. The reference allocates
 * its scratch inside the op with torch::empty (xr64_abs_bridge.cu:160-173); here the
 * caller owns it so the call allocates nothing and can be captured in a CUDA graph. */
size_t xmoe_packed_rows(const xmoe_config* cfg, int32_t n_tokens);
size_t xmoe_workspace_bytes(const xmoe_config* cfg, int32_t n_tokens);
size_t xmoe_workspace_bytes_host_io(const xmoe_config* cfg, int32_t n_tokens);

/* Replaces _C.forward (xr64_abs_bridge.cu:81-232): router -> route pack -> activation
 * quantise+scatter -> FF1 -> FF2 -> combine, ordered on `stream`. N == 0 is a no-op.
 * For batches of at least 4 M elements the activation amax pass runs on a side stream owned by the
 * library (one per device, created on the first such call outside stream capture) and is joined before the
 * quantiser; XMOE_FORK=0 keeps every kernel on the caller's stream. The side stream and its two events exist
 * once per device: forward calls on one device must be serialised by the caller (one host thread, or a lock
 * around the call), or XMOE_FORK=0 must be set. An error return after the fork still joins the side stream. */
int xmoe_forward(const xmoe_config* cfg, const xmoe_weights* w, const void* x, const void* router_logits,
                 int32_t n_tokens, void* y, void* workspace, size_t workspace_bytes, xmoe_stream_t stream);

/* Same call with HOST x / router_logits / y (pinned memory recommended): copies in, runs,
 * copies out and synchronises the stream. Workspace: xmoe_workspace_bytes_host_io. */
int xmoe_forward_host(const xmoe_config* cfg, const xmoe_weights* w, const void* x_host, const void* logits_host,
                      int32_t n_tokens, void* y_host, void* workspace, size_t workspace_bytes, xmoe_stream_t stream);
/* The same without the final synchronisation: copies and kernels are only enqueued on `stream`, and y_host is
 * valid once the caller has synchronised that stream (pinned host memory required for the copies to be
 * asynchronous). A host that keeps two or three calls in flight, each on its own stream with its own workspace
 * and host buffers, overlaps one call's copies with another's kernels: PCIe moves as many bytes per call as the
 * layer takes time, so a serving loop gets about twice the throughput of back-to-back synchronous calls.
 * No reference counterpart (the reference's operator takes device tensors only). */
int xmoe_forward_host_async(const xmoe_config* cfg, const xmoe_weights* w, const void* x_host, const void* logits_host,
                            int32_t n_tokens, void* y_host, void* workspace, size_t workspace_bytes,
                            xmoe_stream_t stream);

/* Synchronises `stream`, then returns the device status word of the last forward on this
 * workspace (0 = ok; 0x100..0x5ff = a bounded device wait gave up, low byte = CTA;
 * 0x600 = an expert id outside [0, E) reached the route pack). */
int xmoe_read_status(const void* workspace, uint32_t* host_out, xmoe_stream_t stream);

/* Variant of _C.forward with routing supplied by the caller, as in the reference's
 * operator(...) (xR64ABSBinding.cu:8-121): topk_idx i32 / topk_w bf16, both [N, top_k].
 * act_scale (device, 3 x f32: XGS, XGSINV, amax) replaces the internal amax pass when not NULL;
 * expert-parallel ranks pass the scale agreed across ranks. */
int xmoe_forward_routed(const xmoe_config* cfg, const xmoe_weights* w, const void* x, const int32_t* topk_idx,
                        const void* topk_w, const float* act_scale, int32_t n_tokens, void* y, void* workspace,
                        size_t workspace_bytes, xmoe_stream_t stream);
/* Same for a buffer of n_tokens rows of which only the first *n_valid_dev (device int32, may be
 * NULL) are in use: the others are neither walked by the route pack nor scanned by the quantiser (their entries
 * of the workspace's index arrays keep whatever an earlier call left there).
 * y may be NULL here and above: the combine is skipped and the FF2 rows stay in the workspace.
 * No reference counterpart (used by the expert-parallel receive path). */
int xmoe_forward_routed_bounded(const xmoe_config* cfg, const xmoe_weights* w, const void* x, const int32_t* topk_idx,
                                const void* topk_w, const float* act_scale, int32_t n_tokens,
                                const int32_t* n_valid_dev, void* y, void* workspace, size_t workspace_bytes,
                                xmoe_stream_t stream);

/* The layer without its combine, the FF2 rows written TOKEN-MAJOR into a caller buffer: rows_out bf16
 * [n_tokens * k_eff, hidden], row (token, slot) at index token * k_eff + slot (k_eff = top_k + num_shared_experts;
 * slots whose expert id is -1 are left untouched). The FF2 epilogue stores there directly, so no gather follows.
 * Routing either from router_logits (topk_idx NULL) or supplied (topk_idx / topk_w as in xmoe_forward_routed);
 * act_scale as there. The caller sums a token's rows itself: xmoe_combine with topk_row[t, s] = t * k_eff + s, or,
 * as the expert-parallel host does for replicated shared experts, lets them land in the buffer that the combine of
 * another exchange already reads. No reference counterpart. */
int xmoe_forward_scatter(const xmoe_config* cfg, const xmoe_weights* w, const void* x, const void* router_logits,
                         const int32_t* topk_idx, const void* topk_w, const float* act_scale, int32_t n_tokens,
                         void* rows_out, void* workspace, size_t workspace_bytes, xmoe_stream_t stream);

/* Per-stage device timing of xmoe_forward* calls, the counterpart of the reference harness's
 * per-kernel timing (sm120a/benchmarks/benchmark.cu:381-399). begin(max_steps > 0) makes every
 * forward record CUDA events between its stages on the caller's stream; read() synchronises
 * the device and returns the summed milliseconds of the 8 stages (router, route pack, amax,
 * quantise, FF1, activation top-k, FF2, combine) over the recorded steps; begin(0) turns it off.
 * Not thread-safe; meant for benchmarks. */
int xmoe_profile_begin(int32_t max_steps);
int xmoe_profile_read(float* stage_ms_sum, int32_t* steps_out);

/* Device pointers into a workspace after a forward, for inspection and tests. */
typedef struct xmoe_workspace_view {
    uint32_t* status;
    float* act_scale;      /* [3]: XGS, XGSINV, amax */
    int32_t* topk_idx;     /* [N, k_eff] */
    void* topk_w;          /* bf16 [N, k_eff] */
    int32_t* topk_off;     /* [N, k_eff] */
    int32_t* topk_row;     /* [N, k_eff] */
    int32_t* counts;       /* [E_tot] */
    int32_t* offsets;      /* [E_tot + 1] */
    int32_t* row_token;    /* [R] */
    void* row_weight;      /* bf16 [R] */
    void* xq;              /* u8 [R, H/2] */
    void* sfx;             /* u8 [R/token_tile, KB, 512] */
    void* yact;            /* bf16 [R, I] */
    void* out_rows;        /* bf16 [R, H] */
    int32_t k_eff;
    int32_t packed_rows;   /* R */
    int32_t kb_pad;        /* KB */
    int32_t token_tile;
} xmoe_workspace_view;
int xmoe_workspace_view_get(const xmoe_config* cfg, int32_t n_tokens, void* workspace, size_t workspace_bytes,
                            xmoe_workspace_view* out);

/* ---- single stages (each replaces one launcher of xR64ABS.cuh:129-199) --------------- */

/* Replaces launch_xr64_abs_topk (xR64ABS.cuh:141-148) / moe_topk_bf16 (sm120a/topk.cuh:25-142).
 * topk_idx / topk_w have row stride idx_stride >= top_k. */
int xmoe_router_topk(const void* router_logits, const float* router_bias, const float* sigmoid_lut,
                     const void* expert_scale, int32_t n_tokens, int32_t num_experts, int32_t top_k,
                     int32_t idx_stride, int32_t scoring, int32_t renormalize, int32_t n_group, int32_t topk_group,
                     float routed_scale, int32_t* topk_idx, void* topk_w, xmoe_stream_t stream);

/* Replaces launch_xr64_abs_route_pack (xR64ABS.cuh:150-160) / moe_route_pack_contiguous
 * (sm120a/preamble.cuh:466-535). scratch: xmoe_route_pack_scratch_bytes. */
size_t xmoe_route_pack_scratch_bytes(int32_t n_tokens, int32_t num_experts, int32_t num_shared);
int xmoe_route_pack(int32_t* topk_idx, void* topk_w, int32_t n_tokens, int32_t num_experts, int32_t top_k,
                    int32_t idx_stride, int32_t num_shared, void* scratch, int32_t* counts, int32_t* offsets,
                    int32_t* topk_off, int32_t* topk_row, int32_t* row_token, void* row_weight, uint32_t* status,
                    xmoe_stream_t stream);

/* No counterpart in the reference. xmoe_route_pack for callers that cannot hand over scratch
 * because they cannot allocate device memory at this point: e.g. a serving engine whose memory
 * pool already owns all free HBM, or a call site where cudaMalloc is unwelcome because it can
 * synchronise the device. The chunk histograms live in a fixed array inside the library
 * (264,192 bytes held by every GPU that loads it, until process exit), so the call allocates
 * nothing: no cudaMalloc / cudaFree and no allocating library routine.
 * Limits: n_tokens <= xmoe_route_pack_static_max_tokens() (16384) and num_experts + num_shared
 * <= 1032; anything larger returns XMOE_ERR_LIMIT and launches nothing.
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress,
 * with that device current): make that first call before any stream capture begins.
 * Every call shares the one array, which keeps the previous call's contents; nothing in it
 * needs clearing (each call rewrites every entry it reads), but two calls that overlap on the
 * GPU - other streams, other host threads - race on it. Outputs are identical to xmoe_route_pack. */
int32_t xmoe_route_pack_static_max_tokens(void);
int xmoe_route_pack_static(int32_t* topk_idx, void* topk_w, int32_t n_tokens, int32_t num_experts, int32_t top_k,
                           int32_t idx_stride, int32_t num_shared, int32_t* counts, int32_t* offsets,
                           int32_t* topk_off, int32_t* topk_row, int32_t* row_token, void* row_weight,
                           uint32_t* status, xmoe_stream_t stream);

/* Replaces moe_act_absmax_partial + moe_act_scale_finalize (sm120a/preamble.cuh:69-128).
 * scratch: 2 x u32, zero on entry (left zero on exit). act_scale: 4 x f32 = XGS, XGSINV, amax, unused. */
int xmoe_act_amax(const void* x, size_t n_elems, uint32_t* scratch, float* act_scale, xmoe_stream_t stream);
/* The finalize half alone (preamble.cuh:98-128): amax (device f32, e.g. after a max all-reduce
 * over expert-parallel ranks) -> act_scale {XGS, XGSINV, amax}. */
int xmoe_act_scale_from_amax(const float* amax, float* act_scale, xmoe_stream_t stream);

/* Replaces launch_xr64_abs_preamble (xR64ABS.cuh:129-139) / moe_act_pack_expert_contiguous
 * (sm120a/preamble.cuh:549-630). */
int xmoe_act_quant_pack(const void* x, const float* act_scale, const int32_t* topk_row, int32_t n_tokens,
                        int32_t hidden, int32_t k_eff, int32_t idx_stride, int32_t token_tile, void* xq, void* sfx,
                        xmoe_stream_t stream);

/* Replaces launch_xr64_abs_ff1 (xR64ABS.cuh:162-176) / xR64FF1 (xR64FF1FF2/xR64FF1.cu:65). */
int xmoe_ff1(const void* w13_packed, const void* w13_sf, const float* w13_gs, const void* xq, const void* sfx,
             const float* act_scale, const int32_t* counts, const int32_t* offsets, const void* row_weight,
             void* yact, uint32_t* status, int32_t e_tot, int32_t hidden, int32_t inter, int32_t packed_rows,
             int32_t token_tile, int32_t activation, float alpha, float limit, xmoe_stream_t stream);

/* No counterpart in the reference: keep the `keep` largest |y| of every FF1 output row. */
int xmoe_act_topk(void* yact, const int32_t* counts, const int32_t* offsets, int32_t e_tot, int32_t inter,
                  int32_t keep, int32_t packed_rows, xmoe_stream_t stream);

/* Replaces launch_xr64_abs_ff2 (xR64ABS.cuh:178-190) / xR64FF2 (xR64FF1FF2/xR64FF2.cu:81),
 * minus its reduce tail: rows stay expert-major. */
int xmoe_ff2(const void* w2_q, const void* w2_scale, const void* yact, const int32_t* counts, const int32_t* offsets,
             void* out_rows, uint32_t* status, int32_t e_tot, int32_t hidden, int32_t inter, int32_t packed_rows,
             int32_t token_tile, xmoe_stream_t stream);

/* Replaces the cp.reduce tail of xR64FF2 / the atomicAdd tail of xR64ABSFF2 plus
 * xR64ABSF32ToBF16 (xr64_abs_bridge.cu:218-229): ordered fp32 sum over the k rows. */
int xmoe_combine(const void* out_rows, const int32_t* topk_row, int32_t n_tokens, int32_t hidden, int32_t k_eff,
                 int32_t idx_stride, void* y, xmoe_stream_t stream);

/* ---- weight preparation (load time) ---------------------------------------------------- */

/* E4M3 block scales [n_mats, rows, K/16] -> MMA scale-factor tiles; out bytes:
 * xmoe_nvfp4_sf_bytes. For w13 pass n_mats = 2*E_tot, rows = I (gate and up are padded
 * to 128 rows separately). No reference counterpart (its layouts are sm_120 fragments). */
size_t xmoe_nvfp4_sf_bytes(int32_t n_mats, int32_t rows, int32_t k);
int xmoe_prep_nvfp4_sf(const void* sf_in, void* sf_out, int32_t n_mats, int32_t rows, int32_t k,
                       xmoe_stream_t stream);

/* Replaces _C.repack_gptq / launch_xr64_abs_repack_gptq (xR64ABS.cuh:192-198, xr64_abs_bridge.cu:61-79,
 * xR64ABSRepack.cu:3-24): GPTQ i32 [E, K/8, O] uint4b8 -> u32 [E, O, K/8]. */
int xmoe_repack_gptq(const void* qweight, void* out, int32_t num_mats, int32_t k, int32_t o, xmoe_stream_t stream);
/* Same target layout from K-major bytes [.., K/2] with low nibble = lower K. */
int xmoe_repack_int4_kmajor(const void* w_in, void* out, size_t n_words, xmoe_stream_t stream);

/* ---- expert parallelism over peer memory (one process per GPU, one node) ---------------- */
/* No counterpart in the reference: its plugin refuses EP != 1 (vllm/xcaliber_int4_vllm/method.py:130-138).
 * Rank g owns routed experts [g * experts_per_rank, (g + 1) * experts_per_rank). Every rank holds the
 * four buffers below, the other ranks map them (CUDA IPC / symmetric memory; the library takes plain
 * device pointers and never opens a handle itself), and the same call sequence runs on every rank's
 * stream with no host synchronisation:
 *   xmoe_ep_post_counts -> xmoe_ep_dispatch -> xmoe_ep_wait_data -> xmoe_forward_routed_bounded (y = NULL, n =
 *   cap_rows, top_k = 1, on recv_x[rank]) -> xmoe_ep_return -> xmoe_ep_wait_ret -> xmoe_combine on
 *   ret_rows[rank]. All device-side waits are bounded (a few seconds; the environment variable
 *   XMOE_EP_SPIN_LIMIT, read at every call, gives a smaller number of ~200 ns polls); a wait that runs out
 *   records XMOE_EP_TIMEOUT and the kernel carries on, so the stream always drains; xmoe_ep_status
 *   reports what went wrong. */
#define XMOE_EP_MAX_WORLD 8
#define XMOE_EP_CTL_BYTES 512
#define XMOE_EP_TIMEOUT 1u   /* a peer's flag did not arrive within the spin limit */
#define XMOE_EP_CAPACITY 2u  /* a row position or home slot fell outside the buffers */
#define XMOE_EP_EXPERT 4u    /* an expert id outside [0, world * experts_per_rank) */
typedef struct xmoe_ep_buffers {
    int32_t world, rank, hidden, experts_per_rank;
    int32_t cap_rows; /* rows of recv_x / recv_meta: worst case world * max_tokens * top_k */
    int32_t ret_cap;  /* rows of ret_rows: >= max_tokens * top_k (+ room the caller uses for shared experts) */
    void* ctl[XMOE_EP_MAX_WORLD];       /* XMOE_EP_CTL_BYTES each, zeroed once before the first call */
    void* recv_x[XMOE_EP_MAX_WORLD];    /* bf16 [cap_rows, hidden] */
    void* recv_meta[XMOE_EP_MAX_WORLD]; /* 16 bytes per row */
    void* ret_rows[XMOE_EP_MAX_WORLD];  /* bf16 [ret_cap, hidden] */
} xmoe_ep_buffers;
/* counts_global: int32 [world * experts_per_rank] rows per expert among this rank's tokens (xmoe_route_pack's
 * counts, run over ALL experts); amax_local: this rank's activation amax (fp32, device) or NULL. */
int xmoe_ep_post_counts(const xmoe_ep_buffers* b, const int32_t* counts_global, const float* amax_local,
                        xmoe_stream_t stream);
/* topk_off = xmoe_route_pack's order inside the expert. amax_global (device fp32, may be NULL) receives the
 * maximum over all ranks' amax_local: feed it to xmoe_act_scale_from_amax. */
int xmoe_ep_dispatch(const xmoe_ep_buffers* b, const void* x, const int32_t* topk_idx, const void* topk_w,
                     const int32_t* topk_off, const int32_t* counts_global, int32_t n_tokens, int32_t top_k,
                     int32_t idx_stride, float* amax_global, xmoe_stream_t stream);
/* e_recv int32 [cap_rows] (local expert id, -1 beyond the received rows), w_recv bf16 [cap_rows], n_recv int32 [1]. */
int xmoe_ep_wait_data(const xmoe_ep_buffers* b, int32_t* e_recv, void* w_recv, int32_t* n_recv,
                      xmoe_stream_t stream);
/* out_rows / topk_row: the local pipeline's FF2 rows and packed-row index per received row (workspace view). */
int xmoe_ep_return(const xmoe_ep_buffers* b, const void* out_rows, const int32_t* topk_row, int32_t expected_rows,
                   xmoe_stream_t stream);
/* The owner-side pipeline with the return transfer fused into FF2: route pack -> quantise -> FF1 -> FF2
 * on recv_x[rank] (cfg: the rank's experts, top_k = 1, no shared experts), where the FF2 epilogue stores
 * every output row straight into its home rank's ret_rows slot and a last tiny kernel raises the return
 * flags. Replaces xmoe_forward_routed_bounded + xmoe_ep_return. row_dst_scratch: 8 bytes per packed row
 * (xmoe_packed_rows(cfg, cap_rows)). quantised_input: 0 = recv_x holds bf16 rows (xmoe_ep_dispatch),
 * 1 = NVFP4 packets (xmoe_ep_dispatch_quantised); act_scale is required in both cases. */
int xmoe_ep_forward_local(const xmoe_ep_buffers* b, const xmoe_config* cfg, const xmoe_weights* w,
                          const int32_t* e_recv, const void* w_recv, const float* act_scale, const int32_t* n_recv_dev,
                          int32_t quantised_input, void* row_dst_scratch, void* workspace, size_t workspace_bytes,
                          xmoe_stream_t stream);
/* xmoe_ep_dispatch fused with the activation quantiser: each token is quantised once on its home GPU with
 * the scale all ranks agree on, and NVFP4 packets travel instead of bf16 rows (3.6x fewer bytes). recv_x[r]
 * then holds codes [cap_rows, hidden/2] followed by block scales [cap_rows, hidden/16]; the owner side runs
 * xmoe_ep_forward_local with quantised_input = 1 (its quantiser becomes a copy). Same packets, bit for bit,
 * as quantising on the owner. */
int xmoe_ep_dispatch_quantised(const xmoe_ep_buffers* b, const void* x, const int32_t* topk_idx, const void* topk_w,
                               const int32_t* topk_off, const int32_t* counts_global, int32_t n_tokens, int32_t top_k,
                               int32_t idx_stride, float* amax_global, xmoe_stream_t stream);
int xmoe_ep_wait_ret(const xmoe_ep_buffers* b, xmoe_stream_t stream);
/* Synchronises the stream and returns the sticky XMOE_EP_* bits of this rank's control block (0 = fine). */
int xmoe_ep_status(const xmoe_ep_buffers* b, xmoe_stream_t stream, uint32_t* bits_out);

/* The step before the layer, done outside the operator in the reference (method.py:255-257 receives
 * router_logits): logits[n, E] = x[n, H] @ gate_w[E, H]^T, bf16 in, fp32 accumulate, bf16 out, on tcgen05.
 * H % 64 == 0, E <= 256. status: a device status word as in the workspace (bounded waits report there). */
int xmoe_gate_logits(const void* x, const void* gate_w, int32_t n_tokens, int32_t hidden, int32_t num_experts,
                     void* logits, uint32_t* status, xmoe_stream_t stream);
/* xmoe_forward with the gate inside: the caller passes x and the router weight gate_w bf16 [num_experts, hidden].
 * ONE kernel runs the gate GEMM and, in its epilogue, the router (bf16 rounding of the logits, top-k, gate
 * weights) straight into the workspace's routing arrays: the same bits as xmoe_gate_logits followed by
 * xmoe_forward, without the logits passing through HBM. logits_out: NULL, or n_tokens * num_experts bf16 that
 * also receive the logits. */
int xmoe_forward_gated(const xmoe_config* cfg, const xmoe_weights* w, const void* x, const void* gate_w,
                       void* logits_out, int32_t n_tokens, void* y, void* workspace, size_t workspace_bytes,
                       xmoe_stream_t stream);

/* Measurement aid, no reference counterpart: the rate at which this GPU retires tcgen05.mma
 * instructions of the largest shape (M 128, N 256) with operands resident on chip, one issuing
 * thread per SM, n_mma instructions each (rounded down to a multiple of 64; ~100000 runs for a
 * few milliseconds). kind 0 = NVFP4 block-scaled (K 64), 1 = bf16 (K 16). Writes dense TFLOP/s
 * of the whole GPU to *tflops_out; synchronises the stream; allocates 4 bytes for the call. */
int xmoe_probe_mma_rate(int32_t kind, int32_t n_mma, double* tflops_out, xmoe_stream_t stream);

/* Host helper: the 65536-entry sigmoid table indexed by bf16 bit pattern. */
void xmoe_fill_sigmoid_lut(float* host_out);

#ifdef __cplusplus
}
#endif
#endif /* XMOE_B200_H_ */
