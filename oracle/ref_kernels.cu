// Thin launch wrappers around the REFERENCE's own router / route-pack / activation
// quantisation kernels, compiled unmodified from the reference tree (the include path is
// given on the nvcc command line by oracle/build_oracle.py; no reference source is copied
// here). TEST INFRASTRUCTURE ONLY: the result, oracle/_ref/libref_kernels.so, is loaded by
// tests/test_gpu_ref_kernels.py on a GPU box to pin the CPU oracle against the reference.
//
// Launch shapes follow the reference harness
// (xFused-NVFP4-Kernels/xMoE/xW4A16/sm120a/benchmarks/benchmark.cu:254-321, 427-432).
#include "preamble.cuh"  // pulls in topk.cuh

extern "C" {

int ref_topk(const uint16_t* logits, int32_t* topk_idx, uint16_t* topk_w, const uint16_t* expert_scale, int n, int e,
             int topk, float routed_scale, int sigmoid, cudaStream_t s) {
    const unsigned grid = ((unsigned)n + 7u) >> 3;
    if (sigmoid)
        moe_topk_bf16<true><<<grid, MOE_TOPK_CTA, 0, s>>>(logits, topk_idx, topk_w, expert_scale, n, e, topk,
                                                          routed_scale);
    else
        moe_topk_bf16<false><<<grid, MOE_TOPK_CTA, 0, s>>>(logits, topk_idx, topk_w, expert_scale, n, e, topk,
                                                           routed_scale);
    return (int)cudaGetLastError();
}

int ref_route_pack(const int32_t* topk_idx, const uint16_t* topk_w, uint16_t* topk_off, uint16_t* expert_topk_w,
                   uint16_t* expert_token_idx, int n, int np, int topk, int e, cudaStream_t s) {
    moe_route_pack_contiguous<<<e, MOE_PREAMBLE_CTA, 0, s>>>(topk_idx, topk_w, topk_off, expert_topk_w,
                                                             expert_token_idx, n, np, topk);
    return (int)cudaGetLastError();
}

// partial: at least `blocks` u32; scale: 8 bytes {float XGS, u32 XGSINV bf16x2}
int ref_act_scale(const uint32_t* x, unsigned long long pairs, uint32_t* partial, unsigned blocks, void* scale,
                  cudaStream_t s) {
    moe_act_absmax_partial<<<blocks, MOE_PREAMBLE_CTA, 0, s>>>(x, pairs, partial);
    moe_act_scale_finalize<<<1, MOE_PREAMBLE_CTA, 0, s>>>(partial, blocks, (MoeActScale*)scale);
    return (int)cudaGetLastError();
}

// X4: u32 [E, NP, H/8]; Sx: u32 [E, NP, H/64]; NP = round_up(N, 32)
int ref_act_pack(const uint32_t* x, const void* scale, const int32_t* topk_idx, const uint16_t* topk_off, uint32_t* x4,
                 uint32_t* sx, int n, int np, int h, int topk, cudaStream_t s) {
    const unsigned grid = (unsigned)(h >> 6) * (unsigned)(np >> 4);
    moe_act_pack_expert_contiguous<<<grid, MOE_PREAMBLE_CTA, 0, s>>>(x, (const MoeActScale*)scale, topk_idx, topk_off,
                                                                     x4, sx, n, np, h, topk);
    return (int)cudaGetLastError();
}

}  // extern "C"
