/*
 * CPU oracle for the EXL3 fused dequant-matmul path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the algorithm of the reference's numpy golden
 * codec `ponyexl3.ref` for one path: packed trellis tile -> 16-bit codewords ->
 * fp16 codebook value -> 16x16 tile -> inner weight matrix, the blockwise
 * 128-point Hadamard rotation with sign vectors, and the linear forward built
 * from them.  It is the parity checker for the CUDA kernels and the timed CPU
 * baseline of the benchmark; the shipped library never links or calls it.
 *
 * Parity is PINNED: tests/golden/ holds vectors produced by importing the
 * reference package itself (tests/golden/make_golden.py), and
 * tests/test_oracle.py checks every function here against them (full 65,536
 * entry tables of all three codebooks by SHA-256, literal per-tile unpack,
 * decoded tiles, and whole forwards).
 *
 * Each function names the reference function it follows (path inside the
 * reference project : lines).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define EXL3O_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ fp16 -- */

static inline float half_bits_to_float(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: renormalise */
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* double -> fp16 bits, round-to-nearest-even in ONE rounding (no intermediate
 * float), as numpy's float16 cast of a Python float does. */
static inline uint16_t double_to_half_bits(double d)
{
    uint64_t b;
    memcpy(&b, &d, 8);
    uint16_t sign = (uint16_t)((b >> 48) & 0x8000u);
    int64_t exp = (int64_t)((b >> 52) & 0x7FF);
    uint64_t man = b & 0xFFFFFFFFFFFFFull;
    if (exp == 0x7FF) return (uint16_t)(sign | 0x7C00u | (man ? 0x200u : 0u));
    if (exp == 0 && man == 0) return sign;
    int64_t e = exp - 1023; /* unbiased */
    if (e > 15) return (uint16_t)(sign | 0x7C00u);
    uint64_t sig = man | (1ull << 52); /* 53-bit significand, value = sig * 2^(e-52) */
    int shift;                         /* bits to drop so that 10 fraction bits stay */
    int64_t he;                        /* resulting biased half exponent */
    if (e >= -14) { shift = 42; he = e + 15; }
    else { shift = (int)(42 + (-14 - e)); he = 0; }
    if (shift > 63) return sign; /* far below the smallest subnormal */
    uint64_t kept = sig >> shift;
    uint64_t rem = sig & ((1ull << shift) - 1);
    uint64_t half = 1ull << (shift - 1);
    if (rem > half || (rem == half && (kept & 1))) kept++;
    /* kept holds the hidden bit (normal) or not (subnormal); a carry out of the
     * mantissa increments the exponent through plain addition. */
    uint32_t out;
    if (he > 0) out = (uint32_t)(((uint64_t)(he - 1) << 10) + kept);
    else out = (uint32_t)kept;
    if (out >= 0x7C00u) out = 0x7C00u;
    return (uint16_t)(sign | out);
}

static inline uint16_t float_to_half_bits(float f) { return double_to_half_bits((double)f); }

/* Exposed so the tests can check the two conversions against numpy. */
EXL3O_API void exl3o_half_to_float(const uint16_t *h, float *f, int64_t n)
{
    for (int64_t i = 0; i < n; i++) f[i] = half_bits_to_float(h[i]);
}
EXL3O_API void exl3o_double_to_half(const double *d, uint16_t *h, int64_t n)
{
    for (int64_t i = 0; i < n; i++) h[i] = double_to_half_bits(d[i]);
}

/* -------------------------------------------------------------- codebook -- */

/* Follows ponyexl3/ref/codebook.py:66-91 (decode_3inst), with lop3_b32 (23-42)
 * taken in its closed form c ^ (a & b) (tests/test_codebook.py:30-31), the
 * half-precision add of the two halves (45-51) and the byte-sum accumulator of
 * vabsdiff4_add (54-63).  cb: 0 = 3INST (default), 1 = MCG, 2 = MUL1. */
EXL3O_API uint16_t exl3o_decode_codeword(uint32_t codeword, int cb)
{
    uint32_t x = codeword & 0xFFFFu;
    if (cb == 0 || cb == 1) {
        if (cb == 0) x = x * 89226354u + 64248484u;
        else x = x * 0xCBAC1FEDu;
        x = (x & 0x8FFF8FFFu) ^ 0x3B603B60u;
        /* Both halves have exponents in [12,15]; their exact sum needs at most
         * 15 significant bits, so it is exact in double and the single rounding
         * below is the correctly rounded fp16 sum. */
        double lo = (double)half_bits_to_float((uint16_t)(x & 0xFFFFu));
        double hi = (double)half_bits_to_float((uint16_t)(x >> 16));
        return double_to_half_bits(lo + hi);
    }
    x = x * 0x83DCD12Du;
    uint32_t s = 0x6400u + (x & 0xFFu) + ((x >> 8) & 0xFFu) + ((x >> 16) & 0xFFu) + (x >> 24);
    double h = (double)half_bits_to_float((uint16_t)(s & 0xFFFFu));
    double k_inv = (double)half_bits_to_float(0x1EEEu);
    double k_bias = (double)half_bits_to_float(0xC931u);
    return double_to_half_bits(h * k_inv + k_bias); /* exact in double, one rounding */
}

EXL3O_API void exl3o_codebook_table(int cb, uint16_t *table65536)
{
    for (uint32_t w = 0; w < 65536u; w++) table65536[w] = exl3o_decode_codeword(w, cb);
}

/* --------------------------------------------------------------- trellis -- */

/* Bit `pos` (0 = first) of the tile's bitstream: the uint16 words are viewed as
 * little-endian uint32 and each uint32 is read from its most significant bit.
 * ponyexl3/ref/trellis.py:121-136 reads the stream through a funnel shift of two
 * such uint32 words; this is the same stream bit by bit. */
static inline uint32_t tile_bit(const uint16_t *packed, int nbits, int pos)
{
    pos %= nbits;
    if (pos < 0) pos += nbits;
    int word32 = pos >> 5;
    int bit_from_msb = pos & 31;
    uint32_t w = (uint32_t)packed[2 * word32] | ((uint32_t)packed[2 * word32 + 1] << 16);
    return (w >> (31 - bit_from_msb)) & 1u;
}

/* Follows ponyexl3/ref/trellis.py:105-141 (unpack_trellis_tile): codeword c is
 * the 16-bit window of the circular 256*K-bit stream that ends at bit (c+1)*K. */
EXL3O_API int exl3o_unpack_tile(const uint16_t *packed, int k, uint16_t *codewords256)
{
    if (k < 1 || k > 8) return -1;
    int nbits = 256 * k;
    for (int c = 0; c < 256; c++) {
        int end = (c + 1) * k;
        uint32_t v = 0;
        for (int b = end - 16; b < end; b++) v = (v << 1) | tile_bit(packed, nbits, b);
        codewords256[c] = (uint16_t)v;
    }
    return 0;
}

/* Follows ponyexl3/ref/trellis.py:12-50 (pack_trellis_tile): the low K bits of
 * each of the 256 values are laid down MSB-first in codeword order. */
EXL3O_API int exl3o_pack_tile(const uint16_t *encoded256, int k, uint16_t *packed)
{
    if (k < 1 || k > 8) return -1;
    int nwords16 = 16 * k;
    memset(packed, 0, (size_t)nwords16 * 2);
    for (int c = 0; c < 256; c++) {
        uint32_t v = encoded256[c] & ((1u << k) - 1u);
        for (int b = 0; b < k; b++) {
            if (!((v >> (k - 1 - b)) & 1u)) continue;
            int pos = c * k + b;
            int word32 = pos >> 5, bit_from_msb = pos & 31;
            int bit = 31 - bit_from_msb; /* bit index inside the LE uint32 */
            int idx16 = 2 * word32 + (bit >> 4);
            packed[idx16] |= (uint16_t)(1u << (bit & 15));
        }
    }
    return 0;
}

/* Tile position (row*16+col) of codeword index i = 8*t + j.  Follows
 * ponyexl3/ref/perm.py:8-26 (tensor_core_perm). */
static inline int tile_pos_of_codeword(int i)
{
    int t = i >> 3, j = i & 7;
    int r0 = (t & 3) * 2;
    int row = r0 + (j & 1) + ((j & 2) ? 8 : 0);
    int col = (t >> 2) + ((j & 4) ? 8 : 0);
    return row * 16 + col;
}

EXL3O_API void exl3o_tile_perm(int32_t *perm256)
{
    for (int i = 0; i < 256; i++) perm256[i] = tile_pos_of_codeword(i);
}

/* Tensor form of the unpack: (n_tiles, 16K) -> (n_tiles, 256).  Follows
 * ponyexl3/ref/trellis.py:205-214 (unpack_trellis). */
EXL3O_API int exl3o_unpack(const uint16_t *packed, int64_t n_tiles, int k, uint16_t *codewords)
{
    if (k < 1 || k > 8) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < n_tiles; t++)
        exl3o_unpack_tile(packed + t * 16 * k, k, codewords + t * 256);
    return 0;
}

/* Fast tile unpack used by the bulk decode: a 64-bit sliding register instead
 * of the bit-by-bit reader.  Checked against exl3o_unpack_tile by the tests. */
static void unpack_tile_fast(const uint16_t *packed, int k, uint16_t *cw)
{
    int nw = 8 * k; /* uint32 words */
    uint32_t words[64];
    for (int i = 0; i < nw; i++)
        words[i] = (uint32_t)packed[2 * i] | ((uint32_t)packed[2 * i + 1] << 16);
    /* state = last 16 bits before position 0 = the stream's final 16 bits */
    uint32_t state = words[nw - 1] & 0xFFFFu;
    int pos = 0;
    for (int c = 0; c < 256; c++) {
        uint32_t fresh = 0;
        for (int b = 0; b < k; b++, pos++)
            fresh = (fresh << 1) | ((words[pos >> 5] >> (31 - (pos & 31))) & 1u);
        state = ((state << k) | fresh) & 0xFFFFu;
        cw[c] = (uint16_t)state;
    }
}

/* Follows ponyexl3/ref/decode.py:32-81 (decode_packed_trellis) and
 * ponyexl3/ref/reconstruct.py:13-23 (reconstruct_inner): the inner weight
 * matrix W (in = 16*t_in rows, ld columns, fp16 bits), tile (tk, tn) at rows
 * 16*tk.., columns 16*(tn - tn0)..; only out-tiles [tn0, tn0+tn_count) are
 * written (the n_offset/n_count column slice of the reference). */
EXL3O_API int exl3o_decode_trellis(const uint16_t *trellis, int64_t t_in, int64_t t_out, int k,
                                   int cb, int64_t tn0, int64_t tn_count, uint16_t *w, int64_t ld)
{
    if (k < 1 || k > 8 || cb < 0 || cb > 2) return -1;
    if (tn0 < 0 || tn0 + tn_count > t_out || ld < 16 * tn_count) return -2;
    uint16_t *table = (uint16_t *)malloc(65536 * 2);
    if (!table) return -3;
    exl3o_codebook_table(cb, table);
    int pos_of[256];
    for (int i = 0; i < 256; i++) pos_of[i] = tile_pos_of_codeword(i);
#pragma omp parallel for schedule(static)
    for (int64_t tk = 0; tk < t_in; tk++) {
        uint16_t cw[256];
        for (int64_t tn = tn0; tn < tn0 + tn_count; tn++) {
            unpack_tile_fast(trellis + (tk * t_out + tn) * 16 * k, k, cw);
            uint16_t *dst = w + (tk * 16) * ld + (tn - tn0) * 16;
            for (int i = 0; i < 256; i++) {
                int p = pos_of[i];
                dst[(p >> 4) * ld + (p & 15)] = table[cw[i]];
            }
        }
    }
    free(table);
    return 0;
}

/* -------------------------------------------------------------- Hadamard -- */

/* Follows ponyexl3/ref/hadamard.py:50-80 (had_r_128): for every 128-wide block
 * of the last dimension, y = ((x * pre) @ H128 / sqrt(128)) * post, H128 the
 * Sylvester matrix (14-23); fp32 in, fp32 out.  The reference evaluates the
 * product as a float32 matmul; here the +-1 sum is taken in double (exact for
 * fp16-valued inputs) and scaled by the float32 constant, which agrees with
 * any float32 summation order to within one float32 ulp.  pre/post are fp16
 * bit patterns or NULL. */
EXL3O_API int exl3o_had128(const float *x, int64_t rows, int64_t n, const uint16_t *pre,
                           const uint16_t *post, float *y)
{
    if (n % 128 != 0) return -1;
    const float scale = (float)(1.0 / sqrt(128.0));
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
        double buf[128];
        for (int64_t j = 0; j < n; j += 128) {
            for (int i = 0; i < 128; i++) {
                float v = x[r * n + j + i];
                if (pre) v = v * half_bits_to_float(pre[j + i]);
                buf[i] = (double)v;
            }
            for (int h = 1; h < 128; h <<= 1)
                for (int i = 0; i < 128; i += 2 * h)
                    for (int q = i; q < i + h; q++) {
                        double a = buf[q], b = buf[q + h];
                        buf[q] = a + b;
                        buf[q + h] = a - b;
                    }
            for (int i = 0; i < 128; i++) {
                float v = (float)(buf[i] * (double)scale);
                if (post) v = v * half_bits_to_float(post[j + i]);
                y[r * n + j + i] = v;
            }
        }
    }
    return 0;
}

/* --------------------------------------------------------------- forward -- */

/* Follows ponyexl3/ref/forward.py:14-49 (linear_forward_reconstruct):
 *   xh = fp16(had(x * suh));  y = fp16(fp32(xh) @ fp32(W));
 *   y  = fp16(had(y) * svh);  y = y + bias (fp16 add).
 * x: (rows, in) fp16 bits; w: (in, out) fp16 bits of the decoded inner matrix;
 * y: (rows, out) fp16 bits.  The float32 dot is accumulated in double and
 * rounded to float32 once, then to fp16 (the reference's float32 matmul result
 * differs from that by at most float32 rounding of partial sums). */
EXL3O_API int exl3o_forward_w(const uint16_t *x, int64_t rows, int64_t in, int64_t out,
                              const uint16_t *w, const uint16_t *suh, const uint16_t *svh,
                              const uint16_t *bias, uint16_t *y)
{
    if (in % 128 || out % 128) return -1;
    float *xf = (float *)malloc(sizeof(float) * rows * in);
    float *xh = (float *)malloc(sizeof(float) * rows * in);
    float *yf = (float *)malloc(sizeof(float) * rows * out);
    float *yh = (float *)malloc(sizeof(float) * rows * out);
    float *wf = (float *)malloc(sizeof(float) * 65536);
    if (!xf || !xh || !yf || !yh || !wf) { free(xf); free(xh); free(yf); free(yh); free(wf); return -3; }
    for (int i = 0; i < 65536; i++) wf[i] = half_bits_to_float((uint16_t)i);
    for (int64_t i = 0; i < rows * in; i++) xf[i] = half_bits_to_float(x[i]);
    exl3o_had128(xf, rows, in, suh, NULL, xh);
    for (int64_t i = 0; i < rows * in; i++) xh[i] = half_bits_to_float(float_to_half_bits(xh[i]));
#pragma omp parallel for schedule(static)
    for (int64_t c0 = 0; c0 < out; c0 += 64) {
        int64_t c1 = c0 + 64 < out ? c0 + 64 : out;
        double acc[64];
        for (int64_t r = 0; r < rows; r++) {
            for (int c = 0; c < 64; c++) acc[c] = 0.0;
            for (int64_t i = 0; i < in; i++) {
                double xv = (double)xh[r * in + i];
                const uint16_t *wr = w + i * out + c0;
                for (int64_t c = 0; c < c1 - c0; c++) acc[c] += xv * (double)wf[wr[c]];
            }
            for (int64_t c = 0; c < c1 - c0; c++)
                yf[r * out + c0 + c] = half_bits_to_float(float_to_half_bits((float)acc[c]));
        }
    }
    exl3o_had128(yf, rows, out, NULL, svh, yh);
    for (int64_t r = 0; r < rows; r++)
        for (int64_t c = 0; c < out; c++) {
            uint16_t h = float_to_half_bits(yh[r * out + c]);
            if (bias) {
                /* numpy's float16 add: float32 sum, then one cast back to fp16 */
                float s = half_bits_to_float(h) + half_bits_to_float(bias[c]);
                h = float_to_half_bits(s);
            }
            y[r * out + c] = h;
        }
    free(xf); free(xh); free(yf); free(yh); free(wf);
    return 0;
}

/* Whole layer forward from the packed trellis (decode + forward_w). */
EXL3O_API int exl3o_forward(const uint16_t *x, int64_t rows, const uint16_t *trellis, int64_t t_in,
                            int64_t t_out, int k, int cb, const uint16_t *suh, const uint16_t *svh,
                            const uint16_t *bias, uint16_t *y)
{
    int64_t in = 16 * t_in, out = 16 * t_out;
    uint16_t *w = (uint16_t *)malloc((size_t)in * out * 2);
    if (!w) return -3;
    int rc = exl3o_decode_trellis(trellis, t_in, t_out, k, cb, 0, t_out, w, out);
    if (rc == 0) rc = exl3o_forward_w(x, rows, in, out, w, suh, svh, bias, y);
    free(w);
    return rc;
}

/* ------------------------------------------------------ trellis encoder -- */

/* One Viterbi pass over the bitshift trellis.  Follows _forward,
 * ponyexl3/convert/reference_search.py:30-57: 65,536 states (16-bit windows), a step appends K
 * bits (s' = ((s << K) | j) & 0xFFFF), so the predecessors of s' are (s' >> K) | (j << (16-K)),
 * j = 0 .. 2^K - 1; float64 costs, the FIRST minimum wins among predecessors and among final
 * states (numpy argmin); branch cost (lut[s'] - w[t])^2 with the product and the sum rounded
 * separately.  back[t][s'] = chosen predecessor.  Returns the best final state. */
static int viterbi_forward(const float *w, int k, const double *lut, int init_state, double *cost, double *next,
                           uint16_t *back)
{
    const int kk = 1 << k;
    for (int s = 0; s < 65536; s++) cost[s] = init_state < 0 ? 0.0 : 1e30;
    if (init_state >= 0) cost[init_state] = 0.0;
    for (int t = 0; t < 256; t++) {
        const double wt = (double)w[t];
        uint16_t *bt = back + (size_t)t * 65536;
#pragma omp parallel for schedule(static)
        for (int s = 0; s < 65536; s++) {
            const uint32_t base = (uint32_t)s >> k;
            uint32_t best = base;
            double cb = cost[base];
            for (int j = 1; j < kk; j++) {
                const uint32_t p = base | ((uint32_t)j << (16 - k));
                if (cost[p] < cb) { cb = cost[p]; best = p; }
            }
            const double d = lut[s] - wt;
            const volatile double d2 = d * d;          /* two roundings, as numpy: no fused multiply-add */
            next[s] = cb + d2;
            bt[s] = (uint16_t)best;
        }
        double *tmp = cost; cost = next; next = tmp;
    }
    int fin = 0;
    for (int s = 1; s < 65536; s++)
        if (cost[s] < cost[fin]) fin = s;
    return fin;
}

/* Exact trellis search of one tile with tail-biting closure.  Follows quantize_tile_reference,
 * ponyexl3/convert/reference_search.py:60-87: a free pass proposes the closing state (the window
 * of codeword 255), pinned passes start from it until the path's pre-state of step 0 and its last
 * state both equal the pin, or max_pins passes are spent.  w: 256 floats in codeword order. */
EXL3O_API int exl3o_quantize_tile(const float *w256, int k, int cb, int max_pins, uint16_t *states256)
{
    if (k < 1 || k > 8 || cb < 0 || cb > 2 || max_pins < 0) return -1;
    double *lut = (double *)malloc(65536 * sizeof(double));
    double *c0 = (double *)malloc(65536 * sizeof(double)), *c1 = (double *)malloc(65536 * sizeof(double));
    uint16_t *back = (uint16_t *)malloc((size_t)256 * 65536 * sizeof(uint16_t));
    if (!lut || !c0 || !c1 || !back) { free(lut); free(c0); free(c1); free(back); return -2; }
    for (uint32_t s = 0; s < 65536u; s++) lut[s] = (double)half_bits_to_float(exl3o_decode_codeword(s, cb));
    int pin = -1, pre0 = 0;
    for (int pass = 0; pass <= max_pins; pass++) {
        int s = viterbi_forward(w256, k, lut, pin, c0, c1, back);
        for (int t = 255; t >= 0; t--) {
            states256[t] = (uint16_t)s;
            s = back[(size_t)t * 65536 + s];
        }
        pre0 = s;
        if (pass > 0 && pre0 == pin && states256[255] == pin) break;
        pin = states256[255];
    }
    free(lut); free(c0); free(c1); free(back);
    return 0;
}

EXL3O_API int exl3o_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

EXL3O_API void exl3o_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
