// Shared device helpers for the sm_100a fused-MoE kernels: status codes, bounded
// mbarrier waits, TMA (cp.async.bulk[.tensor]) issue, tcgen05 (TMEM alloc / MMA /
// commit / ld / cp) wrappers and the UMMA descriptor encoders.
//
// Every wait in this file is bounded: after XMOE_SPIN_LIMIT failed polls the waiter
// records a code in the status word and returns false, so a wrong descriptor or a
// lost transaction shows up as an error code on the host, never as a hung GPU.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>

// ---- status codes returned by the C ABI (0 = ok) ---------------------------------
#define XMOE_OK 0
#define XMOE_ERR_ARG 1        // null pointer / non-positive size
#define XMOE_ERR_SHAPE 2      // shape outside what the kernels support
#define XMOE_ERR_WORKSPACE 3  // workspace too small / misaligned
#define XMOE_ERR_CUDA 4       // a CUDA runtime / driver call failed
#define XMOE_ERR_TIMEOUT 5    // a bounded device-side wait gave up
#define XMOE_ERR_LIMIT 6      // size beyond a stated maximum

// device status word values (written by kernels, read by the host)
#define XMOE_DEV_OK 0u
#define XMOE_DEV_TIMEOUT_TMA 0x100u   // consumer never saw a full stage
#define XMOE_DEV_TIMEOUT_MMA 0x200u   // producer never saw an empty stage
#define XMOE_DEV_TIMEOUT_ACC 0x300u   // epilogue never saw a full accumulator
#define XMOE_DEV_TIMEOUT_EPI 0x400u   // MMA warp never saw a drained accumulator
#define XMOE_DEV_TIMEOUT_DQ 0x500u    // dequant / MMA hand-off wait gave up

// A waiting thread parks inside mbarrier.try_wait for up to XMOE_WAIT_HINT_NS (it wakes as soon
// as the phase completes), so idle roles do not compete for issue slots with the working warps.
// The number of such parked polls is bounded: at most XMOE_SPIN_LIMIT * hint = 2.6 s. The hint is an
// upper limit: on B200 a failed try_wait was seen to return after ~0.5 us, so a wait that is never
// satisfied gives up after ~65 ms at the earliest (the longest legitimate wait, an epilogue warp
// waiting for a whole decode tile, is ~50 us, a few ms under an instrumenting profiler).
#ifndef XMOE_WAIT_HINT_NS
#define XMOE_WAIT_HINT_NS 20000u
#endif
#ifndef XMOE_SPIN_LIMIT
#define XMOE_SPIN_LIMIT (1u << 17)
#endif

namespace xmoe {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31u; }

__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// ---- mbarrier ---------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(XMOE_WAIT_HINT_NS)
        : "memory");
    return ok != 0;
}
// Non-blocking probe of a phase: ~15 cycles when the phase is already complete, where the
// try_wait form with a suspend-time hint costs ~110.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait. Returns false (and records `code` once) when the limit is hit or when
// another role of this CTA has already flagged an error through `abort_flag` (shared).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          uint32_t* status, uint32_t code) {
    if (mbar_test_wait(bar, parity)) return true;  // the common case in a pipeline that runs ahead
    for (uint32_t spin = 0; spin < XMOE_SPIN_LIMIT; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1u;
    if (status) atomicCAS(status, XMOE_DEV_OK, code | (blockIdx.x & 0xffu));
    return false;
}

// ---- TMA --------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* tmap, int x, int y, int z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}
// Untiled bulk copy: both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
// generic-proxy writes (st.shared) -> visible to the async proxy (UMMA / TMA reads)
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- tcgen05 / TMEM ---------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// mbarrier arrives once every tcgen05.mma / tcgen05.cp issued so far by this thread retires.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], block-scaled NVFP4 (E2M1 data, UE4M3 scale per 16 along K), K = 64.
__device__ __forceinline__ void mma_nvfp4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], bf16 x bf16 -> fp32, K = 16.
__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 rows x 16 bytes of shared memory -> 4 TMEM columns, replicated to all 4 lane quadrants
// (the layout block-scaled MMAs read their scale factors from).
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 consecutive fp32 columns: thread t of the warp gets lane (quadrant*32+t).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// ---- UMMA descriptors ---------------------------------------------------------------
// Shared-memory matrix descriptor (64 bit): start>>4 [0,14), LBO>>4 [16,30), SBO>>4 [32,46),
// version=1 [46,48), layout type [61,64) (0 = no swizzle, 2 = 128-byte swizzle).
// K-major, 128-byte swizzle: rows are 128 bytes, 8-row groups are 1024 bytes apart (SBO),
// LBO is not used by the hardware for swizzled K-major tiles (encoded as 1).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)1u << 16;
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1u << 46;
    d |= (uint64_t)2u << 61;
    return d;
}
// No swizzle, one 16-byte column of 8-row core matrices 128 bytes apart: the source
// layout of the 32x128b scale-factor copy.
__device__ __forceinline__ uint64_t umma_desc_sf(uint32_t smem_addr) {
    uint64_t d = (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)(128u >> 4) << 32;
    d |= (uint64_t)1u << 46;
    return d;
}
// Instruction descriptor, block-scaled kinds: a/b format [7,10)/[10,13) (1 = E2M1 for the
// mxf4 kinds), N>>3 [17,23), scale format [23] (0 = UE4M3), M>>4 [24,29). Both operands K-major.
__host__ __device__ constexpr uint32_t umma_idesc_nvfp4(uint32_t m, uint32_t n) {
    return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | (0u << 23) | ((m >> 4) << 24);
}
// Instruction descriptor, kind::f16: accumulator format [4,6) (1 = fp32), a/b format (1 = bf16).
__host__ __device__ constexpr uint32_t umma_idesc_bf16(uint32_t m, uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---- lean issue path -------------------------------------------------------------------
// One thread issues every MMA of a CTA, so the instructions it spends per MMA bound the
// tensor pipe from above (a K=16 bf16 MMA with N=32 lasts ~17 cycles). The helpers below keep
// the 64-bit descriptors as (low word, constant high word): per MMA the issuing thread adds a
// compile-time offset to a 32-bit register and nothing else.
constexpr uint32_t kDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024 B, version 1, 128-byte swizzle
constexpr uint32_t kDescHiSf = (128u >> 4) | (1u << 14);                   // SBO 128 B, version 1, no swizzle
__device__ __forceinline__ uint32_t umma_desc_lo_sw128(uint32_t smem_addr) {
    return ((smem_addr & 0x3ffffu) >> 4) | (1u << 16);
}
__device__ __forceinline__ uint32_t umma_desc_lo_sf(uint32_t smem_addr) { return (smem_addr & 0x3ffffu) >> 4; }

__device__ __forceinline__ void mma_nvfp4_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                             uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %7};\n\t"
        "mov.b64 db, {%2, %7};\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], da, db, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem),
          "r"(kDescHiSw128)
        : "memory");
}
// A from tensor memory (lane = row, 8 columns per K16), B from shared memory.
__device__ __forceinline__ void mma_bf16_ts_lo(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHiSw128)
        : "memory");
}
__device__ __forceinline__ void tmem_cp_sf_lo(uint32_t taddr, uint32_t s_lo) {
    asm volatile(
        "{\n\t.reg .b64 ds;\n\t"
        "mov.b64 ds, {%1, %2};\n\t"
        "tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], ds;\n\t}"
        ::"r"(taddr), "r"(s_lo), "r"(kDescHiSf)
        : "memory");
}

// ---- small numeric helpers ------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t h) { return __uint_as_float(h << 16); }
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float x) {
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(x));
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace xmoe
