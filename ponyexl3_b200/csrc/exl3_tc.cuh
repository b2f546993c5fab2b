// Thin wrappers over the sm_100a tensor-core instructions used by the prefill GEMM:
// tensor-memory allocation, tcgen05.mma with shared-memory descriptors, commit to an
// mbarrier, and tensor-memory loads for the epilogue (cta_group::1; the forms for a pair of
// CTAs are in exl3_gemm2.cuh).
#pragma once
#include <stdint.h>

namespace exl3 {

// ---- tensor memory ---------------------------------------------------------------------------
// Allocate `cols` (power of two >= 32) columns; the base address is written to *smem_dst.
// Executed by all 32 lanes of ONE warp; the same warp frees the columns at the end.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_dst),
                 "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(cols)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync()
{
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync()
{
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
}
// Makes generic-proxy writes to shared memory visible to the tensor core / TMA (async proxy).
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}

// ---- descriptors -----------------------------------------------------------------------------
// Shared-memory matrix descriptor of a K-major operand tile stored in the canonical
// 128-byte-swizzled layout: rows of 64 fp16 (128 bytes), 8-row groups 1024 bytes apart,
// 16-byte chunks XOR-ed with (row & 7).  The tile base must be 1024-byte aligned; a k-step
// of 16 elements inside the 64-wide row advances the start address by 32 bytes.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);   // start address        bits [0,14)
    d |= (uint64_t)1 << 16;                         // leading byte offset (unused here)  [16,30)
    d |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset: 8 rows x 128 B  [32,46)
    d |= (uint64_t)1 << 46;                         // descriptor version of sm_100        [46,48)
    d |= (uint64_t)2 << 61;                         // layout: 128-byte swizzle            [61,64)
    return d;
}

// Instruction descriptor of tcgen05.mma.kind::f16: fp16 A and B (both K-major), fp32 D.
__host__ __device__ constexpr uint32_t mma_idesc_f16(int m, int n)
{
    return (1u << 4)                      // D format: f32
           | (0u << 7) | (0u << 10)       // A, B format: f16
           | (0u << 15) | (0u << 16)      // A, B major: K
           | ((uint32_t)(n >> 3) << 17)   // N / 8
           | ((uint32_t)(m >> 4) << 24);  // M / 16
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The mbarrier gets one arrival when every MMA issued so far by this thread has finished.
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar)
                 : "memory");
}

// 32 consecutive fp32 columns of this thread's tensor-memory lane (warp w reads lanes
// 32*(w%4) .. 32*(w%4)+31).  The wait for the asynchronous load is part of the same asm
// statement, so the compiler can never read the registers before they are written.
__device__ __forceinline__ void tmem_ld_32cols(uint32_t taddr, float (&v)[32])
{
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        "tcgen05.wait::ld.sync.aligned;\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

}  // namespace exl3
