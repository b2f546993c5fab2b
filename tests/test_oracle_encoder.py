"""The oracle's trellis encoder (exact Viterbi search of a tile) against the reference's own
output (tests/golden/encoder.npz, written by make_golden.py from
ponyexl3/convert/reference_search.py) and against the properties the reference's tests check
(tests/test_convert.py:43-58): tail-biting closure, pack / unpack round trip, quantisation error."""

from __future__ import annotations

from pathlib import Path

import numpy as np
import pytest

GOLDEN = Path(__file__).resolve().parent / "golden" / "encoder.npz"


def test_encoder_states_equal_the_reference(oracle):
    g = np.load(GOLDEN)
    for i in range(int(g["n_cases"][0])):
        k, cb = int(g[f"c{i}_k"][0]), int(g[f"c{i}_cb"][0])
        states, decoded = oracle.quantize_tile(g[f"c{i}_w"], k, cb)
        assert (states == g[f"c{i}_states"]).all(), f"case {i}: K={k} cb={cb}"
        assert (decoded == g[f"c{i}_decoded"]).all()


@pytest.mark.parametrize("k", [2, 3])
def test_search_pack_roundtrip(oracle, k):
    w = np.random.default_rng(7).standard_normal(256).astype(np.float32)      # the reference test's tile
    states, decoded = oracle.quantize_tile(w, k)
    s = states.astype(np.uint32)
    nxt = np.roll(s, -1)
    assert ((((s << k) | (nxt & ((1 << k) - 1))) & 0xFFFF) == nxt).all()      # tail-biting transitions
    packed = oracle.pack_trellis_tile((states & ((1 << k) - 1)).astype(np.uint16), k)
    assert (oracle.unpack_trellis_tile(packed, k) == states).all()
    assert float(((decoded - w) ** 2).mean()) < {2: 0.11, 3: 0.032}[k]


def test_encoder_refuses_bad_arguments(oracle):
    with pytest.raises(ValueError):
        oracle.quantize_tile(np.zeros(255, dtype=np.float32), 4)
    with pytest.raises(ValueError):
        oracle.quantize_tile(np.zeros(256, dtype=np.float32), 9)
