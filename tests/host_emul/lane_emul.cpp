// Host build of the kernels' lane arithmetic (ponyexl3_b200/csrc/exl3_bits.cuh):
// runs the per-lane word selection and window extraction for the 32 fragment
// lanes of a tile on the CPU so the tests can compare it with the oracle.
#include <stdint.h>

#include "../../ponyexl3_b200/csrc/exl3_bits.cuh"

namespace {
template <int K> void unpack_tile(const uint32_t* words, uint16_t* cw256)
{
    for (int lane = 0; lane < 32; lane++) {
        exl3::LaneWords<K> lw;
        lw.init(lane);
        uint32_t cw[8];
        exl3::lane_codewords<K>(words[lw.i0], words[lw.i1],
                                exl3::LaneWords<K>::kThree ? words[lw.i2] : 0u, lw.sh, cw);
        for (int j = 0; j < 8; j++) cw256[lane * 8 + j] = (uint16_t)cw[j];
    }
}
}  // namespace

extern "C" int emul_unpack_tile(const uint32_t* words, int k, uint16_t* cw256)
{
    switch (k) {
        case 1: unpack_tile<1>(words, cw256); break;
        case 2: unpack_tile<2>(words, cw256); break;
        case 3: unpack_tile<3>(words, cw256); break;
        case 4: unpack_tile<4>(words, cw256); break;
        case 5: unpack_tile<5>(words, cw256); break;
        case 6: unpack_tile<6>(words, cw256); break;
        case 7: unpack_tile<7>(words, cw256); break;
        case 8: unpack_tile<8>(words, cw256); break;
        default: return -1;
    }
    return 0;
}

// K = 4 fast path: lane t reads word t and word (t - 1) mod 32 of the tile.
extern "C" void emul_unpack_tile_k4_fast(const uint32_t* words, uint16_t* cw256)
{
    for (int lane = 0; lane < 32; lane++) {
        uint32_t cw[8];
        exl3::lane_codewords_k4(words[lane], words[(lane + 31) & 31], cw);
        for (int j = 0; j < 8; j++) cw256[lane * 8 + j] = (uint16_t)cw[j];
    }
}

// Same path with the two 16-bit aligned windows read as halves of the word, as the GEMV does
// with 16-bit shared-memory loads (little-endian: the low half comes first in memory).
extern "C" void emul_unpack_tile_k4_halves(const uint32_t* words, uint16_t* cw256)
{
    const uint16_t* halves = reinterpret_cast<const uint16_t*>(words);
    for (int lane = 0; lane < 32; lane++) {
        uint32_t cw[8];
        exl3::lane_codewords_k4_halves(words[lane], words[(lane + 31) & 31], halves[2 * lane],
                                       halves[2 * lane + 1], cw);
        for (int j = 0; j < 8; j++) cw256[lane * 8 + j] = (uint16_t)cw[j];
    }
}

extern "C" uint32_t emul_codebook_word(int cb, uint32_t cw)
{
    if (cb == 0) return exl3::codebook_word<exl3::CB_3INST>(cw);
    if (cb == 1) return exl3::codebook_word<exl3::CB_MCG>(cw);
    return exl3::codebook_word<exl3::CB_MUL1>(cw);
}

extern "C" void emul_frag_pos(int32_t* pos256)
{
    for (int t = 0; t < 32; t++)
        for (int j = 0; j < 8; j++) pos256[t * 8 + j] = exl3::frag_row(t, j) * 16 + exl3::frag_col(t, j);
}
