// Bit-level pieces of the EXL3 trellis decoder that are plain integer arithmetic:
// which words of a packed tile a fragment lane needs, how the eight 16-bit
// codeword windows are cut out of them, and the integer half of the three
// codebooks.  Everything here compiles for host and device, so the lane
// arithmetic is exercised on the CPU (tests/host_emul) against the oracle
// before any kernel runs.
//
// Tile format (reference: ponyexl3/ref/trellis.py:105-141): a 16x16 tile is
// 256 codewords of K fresh bits each, stored as 8K little-endian uint32 words
// read MSB-first; codeword c is the 16-bit window of that circular 256K-bit
// stream ending at bit (c+1)K.  Codeword index 8t+j belongs to fragment lane t
// (reference: ponyexl3/ref/perm.py:8-26), so lane t needs stream bits
// [8tK + K - 16, 8tK + 8K): 7K+16 bits, at most three words.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define EXL3_HD __host__ __device__ __forceinline__
#else
#define EXL3_HD inline
#endif

namespace exl3 {

enum : int { CB_3INST = 0, CB_MCG = 1, CB_MUL1 = 2 };

// High 32 bits of ((hi:lo) << s), 0 <= s < 32.
EXL3_HD uint32_t funnel_l(uint32_t lo, uint32_t hi, uint32_t s)
{
#if defined(__CUDA_ARCH__)
    return __funnelshift_l(lo, hi, s);
#else
    return s == 0 ? hi : ((hi << s) | (lo >> (32 - s)));
#endif
}

// Which words of its tile a lane reads, and how far its window starts inside
// the first one.  Constant for a lane over the whole kernel.
template <int K> struct LaneWords {
    static constexpr int kWords = 8 * K;          // uint32 words per tile
    static constexpr bool kThree = (K >= 5);      // third word ever needed
    int i0, i1, i2;                               // word indices inside the tile
    uint32_t sh;                                  // bit offset of the window in word i0

    EXL3_HD void init(int lane)
    {
        int p0 = 8 * lane * K + K - 16;           // first stream bit the lane needs
        if (p0 < 0) p0 += 256 * K;                // tail-biting: wraps to the tile's end
        i0 = p0 >> 5;
        sh = (uint32_t)(p0 & 31);
        i1 = i0 + 1; if (i1 >= kWords) i1 -= kWords;
        i2 = i1 + 1; if (i2 >= kWords) i2 -= kWords;
    }
};

// The eight codewords of a lane from its (up to) three words a, b, c, taken in
// stream order.  Output values are zero-extended 16-bit windows.
template <int K> EXL3_HD void lane_codewords(uint32_t a, uint32_t b, uint32_t c, uint32_t sh,
                                             uint32_t (&cw)[8])
{
    // Left-align the lane's 7K+16 bits: n[0] bit 31 is stream bit p0.
    uint32_t n[3];
    n[0] = funnel_l(b, a, sh);
    n[1] = LaneWords<K>::kThree ? funnel_l(c, b, sh) : (b << sh);
    n[2] = LaneWords<K>::kThree ? (c << sh) : 0u;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int off = j * K;                    // window j = bits [off, off+16) of n
        const int q = off >> 5, r = off & 31;
        if (r + 16 <= 32) cw[j] = (n[q] >> (16 - r)) & 0xFFFFu;
        else cw[j] = funnel_l(n[q + 1 > 2 ? 2 : q + 1], n[q], (uint32_t)r) >> 16;
    }
}

// Byte permute of the register pair (b:a) — selector nibble i picks the source byte of
// result byte i (0-3 from a, 4-7 from b).
EXL3_HD uint32_t byte_perm(uint32_t a, uint32_t b, uint32_t sel)
{
#if defined(__CUDA_ARCH__)
    return __byte_perm(a, b, sel);
#else
    const uint64_t v = ((uint64_t)b << 32) | a;
    uint32_t r = 0;
    for (int i = 0; i < 4; i++) r |= (uint32_t)((v >> (8 * ((sel >> (4 * i)) & 7))) & 0xFF) << (8 * i);
    return r;
#endif
}

// 64-bit a * b + (c_hi << 32), returned as (lo, hi).  On the device this is one
// mad.wide.u32, which runs on the integer-multiply pipe and so shifts a word without
// touching the (half-rate) logic/shift pipe.
EXL3_HD void mad_wide(uint32_t a, uint32_t b, uint32_t c_hi, uint32_t& lo, uint32_t& hi)
{
#if defined(__CUDA_ARCH__)
    uint64_t r;
    const uint64_t c = (uint64_t)c_hi << 32;
    asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(r) : "r"(a), "r"(b), "l"(c));
    lo = (uint32_t)r;
    hi = (uint32_t)(r >> 32);
#else
    const uint64_t r = (uint64_t)a * b + ((uint64_t)c_hi << 32);
    lo = (uint32_t)r;
    hi = (uint32_t)(r >> 32);
#endif
}

// K = 4: lane t owns word t of the tile and needs the low 12 bits of word t-1 (its halo).
// With V = (halo : w) as a 44-bit value, codeword j is V >> (28 - 4j) & 0xFFFF.  Odd j are
// byte-aligned in V, even j in V << 4 (one wide multiply); every window is then one byte
// permute with zero fill, and the top one falls out of the wide multiply for free:
// 9 logic-pipe operations for 8 codewords instead of 16 shifts and masks.
// `sixteen` is the number 16 handed in as a run-time value: a literal would be turned back
// into shifts, which run on the quarter-rate shift unit instead of the multiplier.
EXL3_HD void lane_codewords_k4(uint32_t w, uint32_t prev, uint32_t (&cw)[8], uint32_t sixteen = 16u)
{
    const uint32_t p = prev & 0xFFFu;
    uint32_t lo4, hi4;
    mad_wide(w, sixteen, p * sixteen, lo4, hi4);   // (hi4 : lo4) = V << 4, hi4 < 2^16
    cw[7] = byte_perm(w, 0u, 0x4410);
    cw[5] = byte_perm(w, 0u, 0x4421);
    cw[3] = byte_perm(w, 0u, 0x4432);
    cw[1] = byte_perm(w, p, 0x6643);            // w byte 3, halo byte 0, zero, zero
    cw[6] = byte_perm(lo4, 0u, 0x4421);
    cw[4] = byte_perm(lo4, 0u, 0x4432);
    cw[2] = byte_perm(lo4, hi4, 0x6643);
    cw[0] = hi4;
}

// Same, with the two windows that are 16-bit aligned inside the lane's word handed in: w_lo =
// w & 0xFFFF (codeword 7) and w_hi = w >> 16 (codeword 3).  A kernel reads them with 16-bit
// shared-memory loads, which takes two byte permutes per tile off the logic pipe.
EXL3_HD void lane_codewords_k4_halves(uint32_t w, uint32_t prev, uint32_t w_lo, uint32_t w_hi,
                                      uint32_t (&cw)[8], uint32_t sixteen = 16u)
{
    const uint32_t p = prev & 0xFFFu;
    uint32_t lo4, hi4;
    mad_wide(w, sixteen, p * sixteen, lo4, hi4);
    cw[7] = w_lo;
    cw[5] = byte_perm(w, 0u, 0x4421);
    cw[3] = w_hi;
    cw[1] = byte_perm(w, p, 0x6643);
    cw[6] = byte_perm(lo4, 0u, 0x4421);
    cw[4] = byte_perm(lo4, 0u, 0x4432);
    cw[2] = byte_perm(lo4, hi4, 0x6643);
    cw[0] = hi4;
}

// Integer part of the codebooks (reference: ponyexl3/ref/codebook.py:66-91).
// 3INST and MCG: a 32-bit word whose two fp16 halves sum to the weight.
// MUL1: the fp16 bit pattern 0x6400 + (sum of the product's bytes), to be sent
// through one fused multiply-add.
template <int CB> EXL3_HD uint32_t codebook_word(uint32_t cw)
{
    if (CB == CB_MUL1) {
        uint32_t x = cw * 0x83DCD12Du;
#if defined(__CUDA_ARCH__)
        return __dp4a(x, 0x01010101u, 0x6400u);
#else
        return 0x6400u + (x & 0xFFu) + ((x >> 8) & 0xFFu) + ((x >> 16) & 0xFFu) + (x >> 24);
#endif
    }
    uint32_t x = (CB == CB_3INST) ? cw * 89226354u + 64248484u : cw * 0xCBAC1FEDu;
    return (x & 0x8FFF8FFFu) ^ 0x3B603B60u;
}

// Same, with the XOR constant of 3INST / MCG (0x3B603B60) handed in as a run-time value.
// The compiler will not keep a second 32-bit literal in a register and splits (x & m) ^ c
// into two logic operations; a value it cannot see through stays in a register and the
// pair becomes a single three-input LOP3 — one logic-pipe slot per weight saved.
template <int CB> EXL3_HD uint32_t codebook_word_rt(uint32_t cw, uint32_t xor_const)
{
    if (CB == CB_MUL1) return codebook_word<CB>(cw);
    uint32_t x = (CB == CB_3INST) ? cw * 89226354u + 64248484u : cw * 0xCBAC1FEDu;
    return (x & 0x8FFF8FFFu) ^ xor_const;
}

// Tile position (row = input-feature offset, col = output-feature offset) of
// codeword j of lane t (reference: ponyexl3/ref/perm.py:8-26).
EXL3_HD int frag_row(int t, int j) { return (t & 3) * 2 + (j & 1) + ((j & 2) ? 8 : 0); }
EXL3_HD int frag_col(int t, int j) { return (t >> 2) + ((j & 4) ? 8 : 0); }

}  // namespace exl3
