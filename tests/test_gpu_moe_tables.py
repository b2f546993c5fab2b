"""The SwitchGLU table kernels (csrc/exl3_moe.cu) against their host restatement
(tests/test_moe_table_rules.py): decode tables entry by entry, prefill tables through the rules
that do not depend on the order of pairs inside an expert (the kernel's counting sort leaves
that order open)."""

from __future__ import annotations

import numpy as np
import pytest

from test_moe_table_rules import decode_tables, prefill_tables

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from ponyexl3_b200 import _lib
    return _lib


def _routing(n_tokens, top_k, experts, seed):
    rng = np.random.default_rng(seed)
    return np.concatenate([rng.choice(experts, size=top_k, replace=False) for _ in range(n_tokens)])


@pytest.mark.parametrize("lo,hi", [(0, 64), (16, 32), (60, 64)])
@pytest.mark.parametrize("n_tokens", [1, 16])
def test_decode_tables_of_an_expert_range(lib, lo, hi, n_tokens):
    E, kk, D, H = 64, 8, 512, 256
    idx = _routing(n_tokens, kk, E, 5 + n_tokens)
    n = len(idx)
    gb, db = H // 128, D // 128
    d = torch.device("cuda")
    idd = torch.from_numpy(idx).to(d)
    z = lambda *s: torch.full(s, -7, dtype=torch.int32, device=d)
    bgu, bdn, rs, sr, sd, cnt = z(n * 2 * gb, 4), z(n * db, 4), z(2 * n), z(2 * n), z(n), z(2)
    lib.check(lib.load().exl3_moe_decode_tables_range(
        idd.data_ptr(), 8, n, kk, E, lo, hi, D, H, bgu.data_ptr(), rs.data_ptr(), sr.data_ptr(), bdn.data_ptr(),
        sd.data_ptr(), cnt.data_ptr(), 0, torch.cuda.current_stream().cuda_stream), "tables")
    gu, dn, counts = decode_tables(idx.tolist(), lo, hi, D, H)
    assert tuple(cnt.tolist()) == counts
    assert bgu[:counts[0]].tolist() == [list(b) for b in gu]
    assert bdn[:counts[1]].tolist() == [list(b) for b in dn]
    assert bool((bgu[counts[0]:] == -7).all()) and bool((bdn[counts[1]:] == -7).all())   # nothing behind the count
    assert rs.tolist() == [s // kk for s in range(n) for _ in range(2)]
    for s, e in enumerate(idx.tolist()):
        if lo <= e < hi:
            assert sr[2 * s].item() == 2 * (e - lo) and sr[2 * s + 1].item() == 2 * (e - lo) + 1
            assert sd[s].item() == e - lo


@pytest.mark.parametrize("lo,hi", [(0, 16), (4, 8), (12, 16)])
@pytest.mark.parametrize("n_tokens", [96, 700])
def test_prefill_tables_of_an_expert_range(lib, lo, hi, n_tokens):
    E, kk, D, H = 16, 4, 512, 256
    idx = _routing(n_tokens, kk, E, 9 + n_tokens)
    n = len(idx)
    e_here = hi - lo
    slots = n // 256 + e_here
    ct_h, ct_d = (H + 255) // 256, (D + 255) // 256
    d = torch.device("cuda")
    idd = torch.from_numpy(idx).to(d)
    z = lambda *s: torch.full(s, -7, dtype=torch.int32, device=d)
    order, rs, sr, sd, cnt = z(n), z(2 * n), z(2 * n), z(n), z(2)
    tgu, tdn = z(2 * slots * ct_h, 8), z(slots * ct_d, 8)
    lib.check(lib.load().exl3_moe_prefill_tables_range(
        idd.data_ptr(), 8, n, kk, E, lo, hi, D, H, order.data_ptr(), rs.data_ptr(), sr.data_ptr(), sd.data_ptr(),
        tgu.data_ptr(), tdn.data_ptr(), cnt.data_ptr(), 0, torch.cuda.current_stream().cuda_stream), "tables")
    _, _, _, tiles, held = prefill_tables(idx.tolist(), lo, hi)
    assert cnt.tolist() == [2 * held, held]
    got_order = order[:held].tolist()
    assert sorted(got_order) == [s for s, e in enumerate(idx.tolist()) if lo <= e < hi]     # every held pair once
    # an expert's sorted positions are contiguous and in expert order
    experts_sorted = [idx[s] - lo for s in got_order]
    assert experts_sorted == sorted(experts_sorted)
    assert sd[:held].tolist() == experts_sorted
    # rotated rows in use: a prefix, each row's token and sign row belong to its pair
    seg, count = {}, {}
    for pos, e in enumerate(experts_sorted):
        seg.setdefault(e, pos)
        count[e] = count.get(e, 0) + 1
    rs_l, sr_l = rs.tolist(), sr.tolist()
    for pos, s in enumerate(got_order):
        e = experts_sorted[pos]
        i = pos - seg[e]
        rg, ru = 2 * seg[e] + i, 2 * seg[e] + count[e] + i
        assert rs_l[rg] == s // kk and rs_l[ru] == s // kk
        assert sr_l[rg] == 2 * e and sr_l[ru] == 2 * e + 1
    # tiles: the used slots are exactly the restated row tiles; gate tiles then up tiles, shifts as restated
    t_g = tgu[:slots * ct_h].view(slots, ct_h, 8)[:, 0].tolist()
    t_u = tgu[slots * ct_h:].view(slots, ct_h, 8)[:, 0].tolist()
    t_d = tdn.view(slots, ct_d, 8)[:, 0].tolist()
    used = [(g, u, dn) for g, u, dn in zip(t_g, t_u, t_d) if g[0] < g[1]]
    assert len(used) == len(tiles)
    for (g, u, dn), (e, r0, r1, gshift, ushift) in zip(used, tiles):
        assert (g[0], g[1], g[6]) == (r0 + gshift, r1 + gshift, -gshift)
        assert (u[0], u[1], u[6]) == (r0 + ushift, r1 + ushift, -ushift)
        assert (dn[0], dn[1], dn[6]) == (r0, r1, 0)
        assert g[2] == e * (H // 16) and u[2] == (e_here + e) * (H // 16) and dn[2] == e * (D // 16)
    for g, u, dn in zip(t_g[len(tiles):], t_u[len(tiles):], t_d[len(tiles):]):
        assert g[0] >= g[1] and u[0] >= u[1] and dn[0] >= dn[1]                             # unused slots are empty
