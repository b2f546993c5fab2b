"""The item partition of the streamed GEMV (csrc/exl3_gemv.cuh), restated on the host.

The kernel deals the I = blocks x k-blocks items of a layer to G CTAs as contiguous ranges
[I*c/G, I*(c+1)/G) and finishes a column block that straddles CTAs through per-CTA partial
slots and one arrival counter.  These checks pin the integer rules the kernel relies on:
every item belongs to exactly one CTA, `cta_of_item` inverts the range formula, a split block
has one segment per contributor, the slot rule (first segment of a range -> slot 0, else 1)
never puts two live segments of one CTA into one slot, and the counter index (the first
contributor) is unique per split block."""

from __future__ import annotations

import random

import pytest


def cta_of_item(i: int, total: int, grid: int) -> int:
    return ((i + 1) * grid - 1) // total


def segments(c: int, ncb: int, nkb: int, grid: int):
    """(block, first k-block, length, slot) of every segment of CTA c, in processing order."""
    total = ncb * nkb
    i0, i1 = total * c // grid, total * (c + 1) // grid
    out, cur = [], i0
    while cur < i1:
        cb = cur // nkb
        end = min(i1, (cb + 1) * nkb)
        out.append((cb, cur - cb * nkb, end - cur, 0 if cur == i0 else 1))
        cur = end
    return out


CASES = [(136, 40, 296), (40, 136, 296), (40, 40, 296), (1187, 40, 296), (64, 16, 296), (128, 4, 296),
         (1, 136, 136), (3, 1, 3), (5, 7, 4), (1024, 16, 296), (8, 8, 64), (7, 3, 21), (2, 100, 7)]


@pytest.mark.parametrize("ncb,nkb,grid", CASES + [(random.Random(s).randint(1, 300), random.Random(s + 1).randint(1, 150),
                                                    0) for s in range(40)])
def test_partition_rules(ncb, nkb, grid):
    total = ncb * nkb
    if grid == 0:
        grid = min(total, random.Random(ncb * 1000 + nkb).randint(1, 300))
    assert grid <= total
    owner = {}
    for c in range(grid):
        i0, i1 = total * c // grid, total * (c + 1) // grid
        assert i1 > i0                                    # no CTA is empty when grid <= items
        for i in range(i0, i1):
            owner[i] = c
            assert cta_of_item(i, total, grid) == c
    assert len(owner) == total
    counters = {}
    for cb in range(ncb):
        first, last = cb * nkb, cb * nkb + nkb - 1
        cf, cl = cta_of_item(first, total, grid), cta_of_item(last, total, grid)
        contrib = []
        for c in range(cf, cl + 1):
            segs = [s for s in segments(c, ncb, nkb, grid) if s[0] == cb]
            assert len(segs) == 1                         # one segment per contributor
            contrib.append((c, segs[0]))
        assert sum(s[2] for _, s in contrib) == nkb
        if cf == cl:
            assert contrib[0][1][2] == nkb                # complete inside one CTA: no reduction
            continue
        assert cf not in counters                         # the counter index is unique per split block
        counters[cf] = cb
        slot_first = 0 if total * cf // grid == first else 1
        for j, (c, s) in enumerate(contrib):
            assert s[3] == (slot_first if j == 0 else 0)  # the reader's slot rule
    for c in range(grid):
        live = [s[3] for s in segments(c, ncb, nkb, grid) if s[2] < nkb]
        assert len(live) <= 2 and len(set(live)) == len(live)


def effective_grid(items: int, planned: int) -> int:
    """A launch whose block count is read from the device (exl3_gemv_blocks_counted) is planned
    for the table's length; with fewer items than planned CTAs the kernel uses one CTA per item."""
    return max(1, min(planned, items))


@pytest.mark.parametrize("planned", [1, 7, 296])
@pytest.mark.parametrize("nkb", [1, 2, 16])
def test_counted_launch_never_leaves_an_empty_cta_inside_a_split_block(planned, nkb):
    for ncb in list(range(1, 40)) + [296, 297, 1000]:
        total = ncb * nkb
        grid = effective_grid(total, planned)
        assert grid <= total
        for c in range(grid):
            assert total * (c + 1) // grid > total * c // grid
