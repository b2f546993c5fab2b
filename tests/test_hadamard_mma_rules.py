"""The index rules of the tensor-core input rotation (hadamard_mma_kernel, csrc/exl3_basic.cu),
restated on the host: the kernel multiplies 16-row blocks with the 128 x 128 Sylvester matrix as
mma.sync m16n8k16 products whose k index is permuted (a lane loads 8 contiguous columns) and whose
B fragments are built from three sign factors.  This check rebuilds the matrix the kernel
effectively multiplies with from those rules and compares it with H[k][n] = (-1)^popcount(k & n)."""

from __future__ import annotations

import numpy as np


def _parity(v: int) -> int:
    return bin(v).count("1") & 1


def test_fragment_signs_rebuild_the_sylvester_matrix():
    want = np.array([[(-1) ** _parity(k & n) for n in range(128)] for k in range(128)], dtype=np.int64)
    got = np.zeros((128, 128), dtype=np.int64)
    seen = np.zeros((128, 128), dtype=np.int64)
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        # pt[nl][s][j]: two columns (lo, hi) per register
        pt = {}
        for nl in range(4):
            flip = _parity(t & nl)
            for s in range(2):
                for j in range(2):
                    lo = (-1) ** _parity((4 * s + 2 * j) & g)
                    hi = (-1) ** _parity((4 * s + 2 * j + 1) & g)
                    pt[nl, s, j] = ((-1) ** flip * lo, (-1) ** flip * hi)
        for nh in range(4):
            for nl in range(4):
                nt = 4 * nh + nl
                n = 8 * nt + g                        # the B fragment's column is the lane's g
                for q in range(4):
                    acc_sign = -1 if (q & nh) in (1, 2) else 1      # which accumulator the product goes to
                    for s in range(2):                # the two k-steps of a 16-byte load
                        for j in range(2):            # B register 0: k = 2t, 2t+1; register 1: k = 2t+8, 2t+9
                            for half in range(2):
                                k_act = 32 * q + 8 * t + 4 * s + 2 * j + half
                                got[k_act, n] = acc_sign * pt[nl, s, j][half]
                                seen[k_act, n] += 1
    assert (seen == 1).all()                          # every (column, output column) pair is produced exactly once
    assert (got == want).all()


def test_a_fragment_takes_the_columns_the_b_fragment_assumes():
    """A registers of k-step (q, s) of a lane: {row g: h[4s], h[4s+1]}, {row g+8: same},
    {row g: h[4s+2], h[4s+3]}, {row g+8: same}, where h[0..7] are the 8 columns the lane loaded for
    quarter q — i.e. MMA k positions (2t, 2t+1) and (2t+8, 2t+9) hold columns 4s + {0,1} and
    4s + {2,3} of the lane's group, which is what the B fragment's register 0 / register 1 stand for."""
    for t in range(4):
        for q in range(4):
            cols = [32 * q + 8 * t + i for i in range(8)]
            for s in range(2):
                reg0 = cols[4 * s:4 * s + 2]          # xa[q].x (s = 0) or .z (s = 1)
                reg2 = cols[4 * s + 2:4 * s + 4]      # xa[q].y or .w
                assert reg0 == [32 * q + 8 * t + 4 * s, 32 * q + 8 * t + 4 * s + 1]
                assert reg2 == [32 * q + 8 * t + 4 * s + 2, 32 * q + 8 * t + 4 * s + 3]
    # all 128 columns are covered once by the 4 lanes x 4 quarters x 8 columns
    allc = sorted(32 * q + 8 * t + i for q in range(4) for t in range(4) for i in range(8))
    assert allc == list(range(128))
