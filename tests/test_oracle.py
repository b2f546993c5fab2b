"""The CPU oracle against the golden vectors made by the reference itself, plus
the properties the reference's own codec tests check (tests/test_codebook.py,
tests/test_trellis.py, tests/test_decode_reconstruct.py of the reference)."""

from __future__ import annotations

import hashlib

import numpy as np
import pytest

from conftest import rel_err


@pytest.mark.parametrize("cb", [0, 1, 2])
def test_codebook_full_table_matches_reference(oracle, golden, cb):
    table = oracle.codebook_table(cb).view(np.uint16)
    g = golden["codebook"]
    assert hashlib.sha256(table.tobytes()).digest() == g[f"sha256_{cb}"].tobytes()
    np.testing.assert_array_equal(table[::16], g[f"stride16_{cb}"])
    f = table.view(np.float16).astype(np.float64)
    assert np.isfinite(f).all() and np.abs(f).max() < 16.0
    np.testing.assert_allclose([f.min(), f.max(), f.std()], g[f"stats_{cb}"], rtol=1e-12)


def test_codebook_probe_words(oracle, golden):
    g = golden["codebook"]
    for cb in range(3):
        got = np.array([oracle.decode_3inst(int(w), cb) for w in g["probe_words"]])
        np.testing.assert_array_equal(got.view(np.uint16), g["probe_values"][cb])


def test_half_conversions_match_numpy(oracle):
    L = oracle.lib()
    bits = np.arange(65536, dtype=np.uint16)
    f = np.empty(65536, dtype=np.float32)
    L.exl3o_half_to_float(oracle._ptr(bits), oracle._ptr(f), 65536)
    ref = bits.view(np.float16).astype(np.float32)
    np.testing.assert_array_equal(f.view(np.uint32), ref.view(np.uint32))
    rng = np.random.default_rng(0)
    d = np.concatenate([rng.standard_normal(200000) * 10.0 ** rng.integers(-9, 6, 200000),
                        ref.astype(np.float64),
                        (ref[:-1].astype(np.float64) + ref[1:].astype(np.float64)) / 2])
    d = d[np.isfinite(d)]
    h = np.empty(d.size, dtype=np.uint16)
    L.exl3o_double_to_half(oracle._ptr(np.ascontiguousarray(d)), oracle._ptr(h), d.size)
    with np.errstate(over="ignore"):
        want = d.astype(np.float16).view(np.uint16)
    np.testing.assert_array_equal(h, want)


@pytest.mark.parametrize("k", range(1, 9))
def test_unpack_tile_matches_reference(oracle, golden, k):
    g = golden["trellis"]
    for packed, want in zip(g[f"packed_k{k}"], g[f"codewords_k{k}"]):
        np.testing.assert_array_equal(oracle.unpack_trellis_tile(packed, k), want)
    got3 = oracle.unpack_trellis(g[f"packed3_k{k}"], k)
    np.testing.assert_array_equal(got3, g[f"codewords3_k{k}"])


@pytest.mark.parametrize("k", range(1, 9))
def test_pack_matches_reference_and_round_trips(oracle, golden, k):
    g = golden["trellis"]
    enc = g[f"encoded_k{k}"]
    packed = oracle.pack_trellis_tile(enc, k)
    np.testing.assert_array_equal(packed, g[f"encoded_packed_k{k}"])
    np.testing.assert_array_equal(oracle.pack_trellis(g[f"encoded3_k{k}"], k), g[f"packed3_k{k}"])
    mask = (1 << k) - 1
    states = oracle.unpack_trellis_tile(packed, k)
    np.testing.assert_array_equal(states & mask, enc)
    # independent shift-register reconstruction: state' = ((state << K) | fresh) & 0xFFFF
    st, want = 0, np.zeros(256, dtype=np.uint16)
    for t in list(range(256)) * 2:
        st = ((st << k) | int(enc[t])) & 0xFFFF
        want[t] = st
    np.testing.assert_array_equal(states, want)
    keep = (1 << (16 - k)) - 1
    s32 = states.astype(np.uint32)
    assert all(s32[(t + 1) % 256] >> k == (s32[t] & keep) for t in range(256))


def test_perm_matches_reference(oracle, golden):
    np.testing.assert_array_equal(oracle.tensor_core_perm(), golden["trellis"]["perm"])


@pytest.mark.parametrize("k", range(1, 9))
@pytest.mark.parametrize("cb", [0, 1, 2])
def test_decoded_tile_matches_reference(oracle, golden, k, cb):
    g = golden["tiles"]
    packed = g[f"packed_k{k}_cb{cb}"]
    w = oracle.decode_packed_trellis(packed.reshape(1, 1, -1), k, cb)
    assert w.shape == (16, 16) and w.dtype == np.float16
    np.testing.assert_array_equal(w.view(np.uint16), g[f"tile_k{k}_cb{cb}"])


def test_decode_shapes_and_errors(oracle):
    rng = np.random.default_rng(5)
    tr = rng.integers(0, 65536, size=(3, 16, 64), dtype=np.uint16)
    assert oracle.decode_packed_trellis(tr, 4, 0).shape == (48, 256)
    sl = oracle.decode_packed_trellis(tr, 4, 0, n_offset=128, n_count=128)
    np.testing.assert_array_equal(sl, oracle.decode_packed_trellis(tr, 4, 0)[:, 128:])
    with pytest.raises(ValueError):
        oracle.decode_packed_trellis(tr, 3, 0)
    with pytest.raises(ValueError):
        oracle.decode_packed_trellis(tr, 4, 0, n_offset=64)
    with pytest.raises(ValueError):
        oracle.unpack_trellis_tile(np.zeros(10, dtype=np.uint16), 4)
    with pytest.raises(ValueError):
        oracle.pack_trellis_tile(np.zeros(256, dtype=np.uint16), 9)


def test_hadamard_matches_reference(oracle, golden):
    g = golden["hadamard"]
    x = g["x"].view(np.float16).astype(np.float32)
    pre, post = g["pre"].view(np.float16), g["post"].view(np.float16)
    for name, kw in (("y_plain", {}), ("y_pre", dict(pre_scale=pre)), ("y_post", dict(post_scale=post)),
                     ("y_both", dict(pre_scale=pre, post_scale=post))):
        got = oracle.had_r_128(x, **kw)
        np.testing.assert_allclose(got, g[name], rtol=0, atol=2e-6)
    np.testing.assert_array_equal(
        oracle.unpack_sign_bitfield(g["sign_words"].view(np.int16)).view(np.uint16), g["sign_values"])
    with pytest.raises(ValueError):
        oracle.had_r_128(np.zeros((1, 100), dtype=np.float32))


def test_forward_matches_reference(oracle, golden):
    """Decoded weights bit-exact.  Forward outputs equal the reference's except
    where a float32 partial-sum rounding flips one fp16 tie of the pre-rotation
    y; such a flip moves the 128 outputs of its block by at most one fp16 ulp of
    the largest |y|."""
    g = golden["forward"]
    n = int(g["n_cases"][0])
    assert n >= 28
    for i in range(n):
        k, mcg, mul1, inf, outf, rows, has_bias = (int(v) for v in g[f"c{i}_meta"])
        cb = oracle.codebook_mode(bool(mcg), bool(mul1))
        tr = g[f"c{i}_trellis"]
        w = oracle.decode_packed_trellis(tr, k, cb)
        assert hashlib.sha256(np.ascontiguousarray(w).view(np.uint16).tobytes()).digest() == \
            g[f"c{i}_w_sha256"].tobytes(), f"case {i}: decoded weights differ"
        bias = g[f"c{i}_bias"].view(np.float16) if has_bias else None
        x = g[f"c{i}_x"].view(np.float16)
        y = oracle.linear_forward(x, tr, k, cb, g[f"c{i}_suh"].view(np.float16),
                                  g[f"c{i}_svh"].view(np.float16), bias)
        want = g[f"c{i}_y"].view(np.float16)
        assert y.shape == (rows, outf)
        assert rel_err(y, want) < 3e-4, f"case {i}"
        wf = want.astype(np.float64)
        ulp_at_max = float(np.spacing(np.float16(np.abs(wf).max())))
        assert np.abs(y.astype(np.float64) - wf).max() <= ulp_at_max, f"case {i}"


def test_forward_packed_sign_words(oracle, golden):
    g = golden["forward"]
    tr = g["packed_signs_trellis"]
    y = oracle.linear_forward(g["packed_signs_x"].view(np.float16), tr, 3, 0,
                              g["packed_signs_su"], g["packed_signs_sv"])
    assert rel_err(y, g["packed_signs_y"].view(np.float16)) < 3e-4


def test_forward_keeps_leading_shape(oracle):
    rng = np.random.default_rng(3)
    tr = rng.integers(0, 65536, size=(8, 8, 64), dtype=np.uint16)
    y = oracle.linear_forward(np.zeros((2, 3, 128), dtype=np.float16), tr, 4, 0, None, None)
    assert y.shape == (2, 3, 128)
