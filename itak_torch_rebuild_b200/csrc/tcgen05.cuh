// Thin wrappers over the sm_100a tensor-core instructions the multi-row attention kernel uses: tensor-memory
// allocation, tcgen05.mma with shared-memory operand descriptors, completion tracking through an mbarrier,
// and the 32-lane x 32-bit tensor-memory loads / stores.
//
// Shared-memory operand tiles use the 128-byte-swizzle canonical layouts:
//   K-major  (operand rows hold the contraction dimension contiguously): a "panel" is [rows][64 halfs]; row r
//            starts at r * 128 bytes and its 16-byte chunk c sits at chunk (c ^ (r & 7)).  Groups of 8 rows are
//            1024 bytes apart (the descriptor's stride byte offset); one MMA consumes 16 halfs = 32 bytes of every
//            row, so the k-th MMA of a panel starts 32 * k bytes into it.
//   MN-major (operand rows hold the non-contracted dimension contiguously): the same physical panel
//            [k rows][64 halfs], 8 k-rows per 1024-byte group (stride byte offset), panels of the next 64
//            columns one leading byte offset further.
// Every panel starts on a 1024-byte boundary.
#pragma once

#include <stdint.h>

namespace itk {
namespace tc {

// 64-bit shared-memory matrix descriptor: start address, leading / stride byte offsets (all in 16-byte units),
// descriptor version 1 (bits 46-47) and layout type SWIZZLE_128B = 2 (bits 61-63).
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr >> 4) & 0x3fffu);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// 32-bit instruction descriptor of kind::f16 with f16 operands and f32 accumulation: accumulator format f32
// (bits 4-5 = 1), A/B format f16 (0), B major-ness (bit 16: 1 = MN-major), N >> 3 in bits 17-22, M >> 4 in bits 24-28.
__host__ __device__ constexpr uint32_t instr_desc_f16(uint32_t m, uint32_t n, bool b_mn_major) {
    return (1u << 4) | ((b_mn_major ? 1u : 0u) << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot_addr, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_slot_addr), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(cols) : "memory");
}

__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// Generic-proxy writes to shared memory (st.shared, cp.async) become visible to the tensor core's async proxy.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// D(tmem) (+)= A(smem) * B(smem); one thread issues.  accumulate == 0 overwrites D.
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D(tmem) (+)= A(tmem) * B(smem): row i of A lives in tensor-memory lane i, two consecutive f16 elements of the
// contraction dimension per 32-bit column, so one MMA (16 elements) consumes 8 columns starting at a_tmem.
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The mbarrier receives one arrival when every MMA this thread issued before has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar_addr) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar_addr)
                 : "memory");
}

__device__ __forceinline__ void mbar_init(uint32_t bar_addr, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar_addr), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar_addr, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar_addr), "r"(parity)
        : "memory");
    return ok != 0;
}
// Waits for the phase with the given parity for at most `limit_clocks` SM clocks; false = gave up.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar_addr, uint32_t parity, long long limit_clocks) {
    if (mbar_try_wait(bar_addr, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar_addr, parity))
        if (clock64() - t0 > limit_clocks) return false;
    return true;
}

__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// Lane i of the warp reads 16 consecutive 32-bit columns of tensor-memory lane (lane base of taddr) + i.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(
            taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n" ::"r"(taddr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

}  // namespace tc
}  // namespace itk
