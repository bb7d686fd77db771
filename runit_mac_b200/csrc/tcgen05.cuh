// Thin wrappers over the sm_100a tensor-core instructions (tcgen05) and tensor memory (TMEM) used by the
// grouped expert GEMM: allocation, single-thread MMA issue with shared-memory operand descriptors, commit to an
// mbarrier, and accumulator read-back; cta_group::1 (one CTA per tile) and cta_group::2 (a pair of CTAs of one
// cluster shares a 256-row tile: the leader CTA issues the MMAs, each CTA holds half of both operands and its
// 128 accumulator rows).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace runit {

// ── tensor memory ──
// Allocates `cols` columns (power of two, 32..512) of the SM's 128-lane tensor memory; the base address is written
// to shared memory at `holder`.  Executed by one whole warp; the same warp frees it.
__device__ __forceinline__ void tmem_alloc(uint32_t holder, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ── operand descriptors ──
// Shared-memory matrix descriptor of a K-major tile in the 128-byte swizzled layout: rows of 64 16-bit elements
// (128 bytes), groups of 8 rows 1024 bytes apart, 16-byte chunk c of row r stored at chunk position c ^ (r % 8).
// `addr` = shared address of the tile (1024-byte aligned) plus 32 bytes per 16-element K step inside the row.
//   bits  0-13 start address >> 4      bits 16-29 leading byte offset >> 4 (unused for swizzled K-major: 1)
//   bits 32-45 stride byte offset >> 4 (1024 >> 4)      bits 46-47 descriptor version (1 on sm_100)
//   bits 61-63 layout (2 = 128-byte swizzle)
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor for kind::f16 with bf16 A and B (both K-major), f32 accumulator, tile M x N.
//   bits 4-5 D format (1 = f32)   bits 7-9 A format (1 = bf16)   bits 10-12 B format (1 = bf16)
//   bit 15 / 16 A / B major (0 = K)   bits 17-22 N >> 3   bits 24-28 M >> 4
__host__ __device__ constexpr uint32_t umma_idesc_bf16(uint32_t m, uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T, issued by ONE thread.  accumulate == 0 overwrites D.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(d_tmem), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The mbarrier receives one arrival when every MMA issued so far by this thread has completed
// (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ── accumulator read-back: 32 consecutive columns of this warp's 32 lanes (lane i of the warp reads TMEM lane
//    (taddr.lane + i)); a warp may only touch the lane quarter 32*(warp index % 4).  Whole warp. ──
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ── mbarrier helpers for the warp-specialised pipeline ──
constexpr uint32_t kSuspendHintNs = 200000;   // upper bound of one try_wait; the timed loops re-check abort and clock between tries
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t done;
    // The suspend-time hint (ns) lets the hardware park the thread until the phase completes; without it the
    // instruction returns almost at once and a waiting role burns the issue slots of the warps that do the work.
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(done)
                 : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
                 : "memory");
    return done != 0;
}
// Wait bounded by time (2^31 SM cycles, about a second) and by the CTA's abort flag: returns false when the wait gave
// up; the first thread to give up raises the flag so that every other role of the CTA leaves its loop too.  The
// cycle counter is read once per 8 failed polls (each poll suspends the thread for up to kSuspendHintNs).
__device__ __forceinline__ bool mbar_wait_timed(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 8; i++)
            if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > (1ll << 31)) {
            *abort_flag = 1;
            return false;
        }
    }
}

// ───────────────────────── CTA pairs (cta_group::2) ─────────────────────────
// Allocation and release are executed by the same warp index in BOTH CTAs of the pair, with the same holder offset.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t holder, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// Issued by one thread of the leader CTA; both CTAs' shared-memory tiles sit at the offsets the descriptors name.
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(d_tmem), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One arrival on the mbarrier at this shared-memory offset in every CTA of `cta_mask` once the MMAs issued so far
// have completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(cta_mask)
                 : "memory");
}
// Same with the A operand in tensor memory (128 lanes per CTA, 32-bit column c of the operand = K elements 2c, 2c+1).
__device__ __forceinline__ void umma_bf16_pair_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Registers -> tensor memory: 16 consecutive columns of this warp's 32 lanes (whole warp; the lane quarter rule of
// tmem_ld32 applies).  tmem_st_wait makes the stores of the executing thread complete.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Address of a shared-memory location of CTA `rank` of the cluster, in the cluster-wide shared window.
__device__ __forceinline__ uint32_t cluster_map(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
// Arrival on an mbarrier of another CTA of the cluster (address from cluster_map).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_cluster(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(done)
                 : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
                 : "memory");
    return done != 0;
}
// Same bounded wait, for barriers that threads of the peer CTA arrive on.  (Cluster-scope release/acquire
// qualifiers on the arrive and the wait were measured to cost about 1500 cycles per remote arrival; the default
// semantics, which the dequantisers' proxy fence completes, are the ones used.)
__device__ __forceinline__ bool mbar_wait_timed_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 8; i++)
            if (mbar_try_cluster(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > (1ll << 31)) {
            *abort_flag = 1;
            return false;
        }
    }
}
// 2-D tiled load into this CTA's shared memory whose completion bytes are counted on an mbarrier of the pair's
// leader CTA (`bar_cluster_addr` from cluster_map); no data is shared between the CTAs by this load.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int32_t c0, int32_t c1, uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar_cluster_addr)
        : "memory");
}

}  // namespace runit
