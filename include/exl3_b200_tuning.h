/*
 * exl3_b200_tuning — benchmark knobs of libexl3b200.so, outside the stable ABI of exl3_b200.h.
 *
 * These set process-wide state that every later streamed-GEMV launch reads; they exist for
 * sweeps that look for the best launch shape and are never called on a product path.  They have
 * no counterpart in the reference.
 */
#ifndef EXL3_B200_TUNING_H
#define EXL3_B200_TUNING_H

#include "exl3_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* max_grid: largest number of virtual CTAs (halves of the 1024-thread CTAs) a streamed GEMV
 * deals its items to (0 = two per SM, the default);
 * fuse_x_bytes: the input rotation runs inside the GEMV when the rotated words of one half fit in
 * this many bytes of shared memory, 0 .. 28,672 (values outside leave it as it is; the default
 * is the maximum; 0 always uses the separate rotation kernel). */
EXL3_API void exl3_tune_gemv(int max_grid, int fuse_x_bytes);

/* one_acc_rows: 128 (default) = an output tile of the prefill GEMM with at most 128 rows loads,
 * multiplies and drains only its first accumulator; 0 = every tile uses both (for comparison).
 * + 256: a dense layer's short last wave of tiles is NOT cut into 128-column half tiles. */
EXL3_API void exl3_tune_gemm(int one_acc_rows);

/* on: 1 = dense prefill GEMMs of 1024 rows and more run on pairs of SMs
 * (tcgen05.mma.cta_group::2, 512-row output tiles); 0 (default) = the one-CTA kernel for every
 * shape, which is a little faster on the shapes measured so far. */
EXL3_API void exl3_tune_gemm_pairs(int on);

#ifdef __cplusplus
}
#endif
#endif /* EXL3_B200_TUNING_H */
