"""The launch tables of the stacked-expert SwitchGLU (csrc/exl3_moe.cu), restated on the host.

The kernels turn routing indices into block tables (few tokens) and tile tables (many tokens),
optionally for a GPU that holds only a range of the experts.  These checks pin the integer rules
the GEMV / GEMM launches rely on: held pairs are packed to the front in pair order and counted;
an expert's rotated gate rows and up rows lie next to each other, so the rows in use are a prefix;
a row tile never straddles two experts; a tile's row shift maps its rotated rows back to the
sorted position; and the ranks' shares partition the pairs."""

from __future__ import annotations

import numpy as np
import pytest


def decode_tables(idx, lo, hi, D, H):
    """(blocks_gu, blocks_dn, counts) for the experts lo..hi-1; block = (phys, xrow, sv_off, y_off)."""
    gb, db, e_here = H // 128, D // 128, hi - lo
    held = [(s, e - lo) for s, e in enumerate(idx) if lo <= e < hi]
    gu, dn = [], []
    for q, (s, el) in enumerate(held):
        for p in range(2):
            for j in range(gb):
                gu.append(((p * e_here + el) * gb + j, 2 * s + p, el * 2 * H + p * H + 128 * j, s * 2 * H + p * H + 128 * j))
        for j in range(db):
            dn.append((el * db + j, s, el * D + 128 * j, s * D + 128 * j))
    return gu, dn, (len(held) * 2 * gb, len(held) * db)


def prefill_tables(idx, lo, hi):
    """Sorted order, rotated-row owners and row tiles for the experts lo..hi-1."""
    e_here = hi - lo
    local = [e - lo if lo <= e < hi else -1 for e in idx]
    count = [sum(1 for e in local if e == x) for x in range(e_here)]
    seg = np.concatenate([[0], np.cumsum(count)])[:-1].tolist()
    order, cursor = {}, [0] * e_here
    gate_row, up_row = {}, {}
    for s, e in enumerate(local):
        if e < 0:
            continue
        i = cursor[e]
        cursor[e] += 1
        order[seg[e] + i] = s
        gate_row[s] = 2 * seg[e] + i
        up_row[s] = 2 * seg[e] + count[e] + i
    tiles = []                     # (expert, row0, row_end, gate shift, up shift) in sorted positions
    for e in range(e_here):
        for b in range((count[e] + 255) // 256):
            r0 = seg[e] + 256 * b
            tiles.append((e, r0, min(r0 + 256, seg[e] + count[e]), seg[e], seg[e] + count[e]))
    return order, gate_row, up_row, tiles, sum(count)


@pytest.mark.parametrize("world", [1, 2, 3, 8])
@pytest.mark.parametrize("n_tokens,top_k,experts", [(1, 8, 256), (16, 8, 256), (5, 2, 8)])
def test_decode_blocks_of_all_ranks_partition_the_pairs(world, n_tokens, top_k, experts):
    rng = np.random.default_rng(n_tokens * 100 + world)
    idx = np.concatenate([rng.choice(experts, size=top_k, replace=False) for _ in range(n_tokens)]).tolist()
    D, H = 2048, 512
    seen_gu, seen_dn = set(), set()
    for rank in range(world):
        base, extra = divmod(experts, world)
        lo = rank * base + min(rank, extra)
        hi = lo + base + (1 if rank < extra else 0)
        gu, dn, counts = decode_tables(idx, lo, hi, D, H)
        assert counts == (len(gu), len(dn))
        rows = [b[1] for b in gu]
        assert rows == sorted(rows)                                   # pair order is kept
        for phys, xrow, sv, yo in gu:
            assert 0 <= phys < 2 * (hi - lo) * (H // 128) and 0 <= sv < (hi - lo) * 2 * H
            assert (xrow, yo) not in seen_gu
            seen_gu.add((xrow, yo))
        for phys, xrow, sv, yo in dn:
            assert 0 <= phys < (hi - lo) * (D // 128) and 0 <= sv < (hi - lo) * D
            assert (xrow, yo) not in seen_dn
            seen_dn.add((xrow, yo))
    n = len(idx)
    assert len(seen_gu) == n * 2 * (H // 128) and len(seen_dn) == n * (D // 128)


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("n_tokens,top_k,experts", [(96, 4, 16), (700, 2, 8), (40, 8, 64)])
def test_prefill_rows_and_tiles(world, n_tokens, top_k, experts):
    rng = np.random.default_rng(n_tokens + world)
    idx = np.concatenate([rng.choice(experts, size=top_k, replace=False) for _ in range(n_tokens)]).tolist()
    all_pairs = []
    for rank in range(world):
        base, extra = divmod(experts, world)
        lo = rank * base + min(rank, extra)
        hi = lo + base + (1 if rank < extra else 0)
        order, gate_row, up_row, tiles, held = prefill_tables(idx, lo, hi)
        assert sorted(order) == list(range(held))                     # sorted positions are a prefix
        rows = sorted(list(gate_row.values()) + list(up_row.values()))
        assert rows == list(range(2 * held))                          # rotated rows in use are a prefix
        covered = []
        for e, r0, r1, gshift, ushift in tiles:
            assert 0 < r1 - r0 <= 256
            for pos in range(r0, r1):
                s = order[pos]
                assert idx[s] - lo == e                               # a tile never straddles two experts
                assert gate_row[s] == pos + gshift and up_row[s] == pos + ushift   # row - shift = sorted position
                covered.append(pos)
        assert sorted(covered) == list(range(held))
        all_pairs += list(order.values())
    assert sorted(all_pairs) == list(range(len(idx)))                 # the ranks' shares partition the pairs
