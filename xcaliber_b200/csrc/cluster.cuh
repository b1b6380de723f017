// Helpers for kernels that run as clusters of two CTAs and issue 2-SM MMAs (tcgen05
// cta_group::2): peer addressing, remote mbarrier arrives, cluster-scope bounded waits, paired
// tensor-memory allocation and commits that target either CTA's barrier (or, with an arrival
// mask, the same barrier in both). No data is ever multicast: every TMA load is a plain local load.
#pragma once

#include "common.cuh"

namespace xmoe {

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of `local_smem_addr` in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_smem_addr), "r"(rank));
    return a;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Bounded wait on a barrier that also receives arrivals from the peer CTA. The waiting thread
// never reads data the peer wrote with ordinary stores: the remote arrivals only announce that
// TMA data / tensor-memory data of the peer are in place for the 2-SM MMA, or that the peer is
// done with a buffer. A CTA-scope wait is therefore enough.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                                  uint32_t* status, uint32_t code) {
    return mbar_wait(bar, parity, abort_flag, status, code);
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Arrive on the barrier at `cluster_addr` (either CTA of the pair) once all MMAs / copies issued
// so far by this thread retire.
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
                 : "memory");
}
// Same, arriving on the barrier at the same shared-memory offset in every CTA of `cta_mask`
// (bit i = CTA rank i of the cluster): one instruction instead of one commit per CTA. This is a
// multicast of the ARRIVAL only; no data is multicast.
__device__ __forceinline__ void tc_commit_pair_mask(uint32_t local_addr, uint16_t cta_mask) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(local_addr), "h"(cta_mask)
        : "memory");
}
// 2-SM block-scaled NVFP4 MMA: D (256 x N; 128 rows in each CTA's tensor memory) (+)= A (128 rows
// from each CTA's shared memory) * B (N/2 rows from each CTA's shared memory, same offsets);
// scale factors of A (own rows) and of all of B must sit in each CTA's tensor memory.
__device__ __forceinline__ void mma_nvfp4_pair(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                               uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %7};\n\t"
        "mov.b64 db, {%2, %7};\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], da, db, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem),
          "r"(kDescHiSw128)
        : "memory");
}
// Scale-factor copy issued once for the pair: each CTA's shared memory (same offset) -> its own
// tensor memory (same column).
__device__ __forceinline__ void tmem_cp_sf_pair(uint32_t taddr, uint32_t s_lo) {
    asm volatile(
        "{\n\t.reg .b64 ds;\n\t"
        "mov.b64 ds, {%1, %2};\n\t"
        "tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], ds;\n\t}"
        ::"r"(taddr), "r"(s_lo), "r"(kDescHiSf)
        : "memory");
}

}  // namespace xmoe
