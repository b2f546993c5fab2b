// Device-only building blocks shared by the kernels: exact fp16 codebook
// arithmetic, the m16n8k16 fragment multiply, the 128-point Hadamard butterfly
// of one warp, and thin wrappers over the sm_100a asynchronous-copy / mbarrier /
// programmatic-launch instructions.  Every wait on an mbarrier is bounded.
#pragma once
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "exl3_bits.cuh"

namespace exl3 {

// Status bits a kernel may set in the workspace status word.
enum : int {
    ST_WAIT_FULL_TIMEOUT = 1,    // a consumer gave up waiting for a staged item
    ST_WAIT_EMPTY_TIMEOUT = 2,   // the producer gave up waiting for a free stage
    ST_TC_TIMEOUT = 4,           // a tensor-core pipeline wait gave up
    ST_BAD_LAUNCH = 8,           // a kernel found its launch (shared memory, cluster) not as planned
    ST_PEER_TIMEOUT = 16,        // a wait for the other GPUs' output blocks gave up
};

// ---- codebooks: exact fp16 arithmetic -------------------------------------------------

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// Two codewords -> one register holding (w_a, w_b) as fp16, bit-exact with the
// reference codebooks (ponyexl3/ref/codebook.py:66-91): 3INST / MCG add the two
// fp16 halves of the scrambled word with one rounding; MUL1 sends the fp16
// pattern 0x6400 + byte-sum through one fused multiply-add.
template <int CB> __device__ __forceinline__ uint32_t decode_pair(uint32_t cw_a, uint32_t cw_b)
{
    const uint32_t xa = codebook_word<CB>(cw_a);
    const uint32_t xb = codebook_word<CB>(cw_b);
    if (CB == CB_MUL1) {
        const uint32_t s = xa | (xb << 16);
        const __half2 kinv = u32_as_h2(0x1EEE1EEEu), kbias = u32_as_h2(0xC931C931u);
        return h2_as_u32(__hfma2(u32_as_h2(s), kinv, kbias));
    }
    const uint32_t lo = __byte_perm(xa, xb, 0x5410);   // (lo_a, lo_b)
    const uint32_t hi = __byte_perm(xa, xb, 0x7632);   // (hi_a, hi_b)
    return h2_as_u32(__hadd2(u32_as_h2(lo), u32_as_h2(hi)));
}

template <int CB> __device__ __forceinline__ __half decode_one(uint32_t cw)
{
    return __low2half(u32_as_h2(decode_pair<CB>(cw, cw)));
}

// ---- tensor-core fragment multiply ------------------------------------------------------

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col).  The packed tile order of
// EXL3 is exactly the A-fragment order of W^T (out x in), so decoded registers feed
// this directly (a0: codewords 0,1; a1: 4,5; a2: 2,3; a3: 6,7 of the lane).
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ---- Hadamard ---------------------------------------------------------------------------

// In-place 128-point Sylvester Hadamard of a block spread over one warp, lane l
// holding elements 4l..4l+3; un-normalised (caller scales by 1/sqrt(128)).
__device__ __forceinline__ void had128_warp(float (&v)[4], int lane)
{
    float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
    v[0] = a + c; v[1] = b + d; v[2] = a - c; v[3] = b - d;
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
        const bool upper = (lane & m) != 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float o = __shfl_xor_sync(0xFFFFFFFFu, v[i], m);
            v[i] = upper ? (o - v[i]) : (v[i] + o);
        }
    }
}

#define EXL3_HAD_SCALE 0.08838834764831845f

// ---- gated linear unit ------------------------------------------------------------------------

// act(g) * u in fp32 (the caller rounds to fp16): mode 1 = SiLU, 2 = tanh-GELU, the two
// activations of the reference's SwitchGLU (ponyexl3/mlx/exl3_moe.py:62-75).
enum : int { GLU_NONE = 0, GLU_SILU = 1, GLU_GELU = 2 };
__device__ __forceinline__ float glu_value(float g, float u, int mode)
{
    if (mode == GLU_GELU)
        return 0.5f * g * (1.f + tanhf(0.797884560803f * (g + 0.044715f * g * g * g))) * u;
    return g / (1.f + __expf(-g)) * u;
}

// ---- shared-memory barriers and bulk copies ------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: false after kWaitSpins unsuccessful polls (each poll already
// blocks for a hardware-defined interval).
constexpr uint32_t kWaitSpins = 1u << 20;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity)
{
    for (uint32_t i = 0; i < kWaitSpins; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// Contiguous global -> shared copy by the bulk-copy engine; both addresses 16-byte
// aligned, size a multiple of 16.  Completion is counted on `bar` in bytes.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::
            "r"(dst), "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

// Programmatic dependent launch: let the next kernel of the stream start its
// independent prologue / wait until the kernels this one depends on have finished.
__device__ __forceinline__ void griddep_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

__device__ __forceinline__ void named_bar_sync(int id, int threads)
{
    asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ float ld_cg_f32(const float* p)
{
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];\n" : "=f"(v) : "l"(p));
    return v;
}

}  // namespace exl3
