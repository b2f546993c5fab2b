"""The CUDA trellis encoder (exl3_encode_tiles) through the C ABI: states bit-identical to the
reference's search (golden vectors) and to the oracle on random tiles, packed tiles that unpack
to the same states and decode to the codebook values of those states, and a whole matrix
quantised and decoded again."""

from __future__ import annotations

from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

GOLDEN = Path(__file__).resolve().parent / "golden" / "encoder.npz"


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from ponyexl3_b200 import ops
    return ops


def _u16(t):
    return t.cpu().numpy().view(np.uint16)


def test_encoder_states_equal_the_reference(ops):
    g = np.load(GOLDEN)
    for i in range(int(g["n_cases"][0])):
        k, cb = int(g[f"c{i}_k"][0]), int(g[f"c{i}_cb"][0])
        states, packed = ops.quantize_tiles(torch.from_numpy(g[f"c{i}_w"]).cuda().view(1, 256), k, cb)
        assert (_u16(states)[0] == g[f"c{i}_states"]).all(), f"case {i}: K={k} cb={cb}"
        assert (_u16(ops.unpack_trellis(packed.view(1, 1, 16 * k), k))[0, 0] == g[f"c{i}_states"]).all()


@pytest.mark.parametrize("k,cb", [(2, 0), (3, 1), (4, 0), (4, 2)])
def test_encoder_matches_the_oracle_on_random_tiles(ops, oracle, k, cb):
    rng = np.random.default_rng(100 + 10 * k + cb)
    w = (rng.standard_normal((5, 256)) * rng.uniform(0.3, 2.0, size=(5, 1))).astype(np.float32)
    states, packed = ops.quantize_tiles(torch.from_numpy(w).cuda(), k, cb, max_tiles_in_flight=3)   # tiles share slots
    got = _u16(states)
    for t in range(5):
        want, _ = oracle.quantize_tile(w[t], k, cb)
        assert (got[t] == want).all(), f"tile {t}"
        assert (_u16(packed)[t] == oracle.pack_trellis_tile((want & ((1 << k) - 1)).astype(np.uint16), k)).all()


def test_quantised_matrix_decodes_to_the_chosen_codebook_values(ops, oracle):
    k, cb = 3, 0
    rng = np.random.default_rng(3)
    inner = rng.standard_normal((32, 48)).astype(np.float32)
    trellis = ops.quantize_inner(torch.from_numpy(inner).cuda(), k, cb)
    assert tuple(trellis.shape) == (2, 3, 16 * k)
    w = ops.decode_packed_trellis(trellis, k, cb).float().cpu().numpy()
    assert w.shape == inner.shape
    assert float(((w - inner) ** 2).mean()) < 0.032            # the reference test's bound for K = 3
    # one tile against the oracle's search of the same tile in codeword order
    perm = oracle.tensor_core_perm()
    tile = inner[16:32, 16:32].reshape(256)[perm]
    _, decoded = oracle.quantize_tile(tile, k, cb)
    assert (w[16:32, 16:32].reshape(256)[perm] == decoded).all()
