// tcgen05 (5th-generation tensor core) PTX wrappers shared by the sm_100a kernels of this folder:
// fences around thread synchronisation, the commit that signals an mbarrier when the products issued so
// far are done, products with the first operand in shared or in tensor memory, and the shared-memory
// operand descriptors for 128-byte-swizzled tiles.
#pragma once

#include <stdint.h>

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem] . B[smem]
__device__ __forceinline__ void tc_mma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
// D[tmem] (+)= A[tmem] . B[smem]
__device__ __forceinline__ void tc_mma_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d), "r"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}

// Shared-memory operand descriptors.  Bits: [0,14) address>>4, [16,30) leading offset>>4, [32,46) stride
// offset>>4, [46,48) version 1, [61,64) layout 2 (128-byte swizzle).
// K-major operand: rows of 128 bytes, groups of eight rows 1024 bytes apart (the leading offset is unused, 1).
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// MN-major operand: 64 contiguous elements of the N dimension per 128-byte row, one row per k; eight-k groups
// 1024 bytes apart (stride offset), the next 64 elements of N `chunk_bytes` further (leading offset).
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t chunk_bytes) {
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((chunk_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
