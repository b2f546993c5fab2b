"""The kernels' per-lane integer arithmetic, compiled for the host and compared
with the oracle: which words of a packed tile each fragment lane reads, the
eight codeword windows it cuts out of them (all K), the integer half of the
three codebooks (all 65,536 codewords) and the fragment position table."""

from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np
import pytest

HERE = Path(__file__).resolve().parent


@pytest.fixture(scope="module")
def emul(tmp_path_factory):
    out = tmp_path_factory.mktemp("emul") / "liblane_emul.so"
    subprocess.run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-o", str(out),
                    str(HERE / "host_emul" / "lane_emul.cpp")], check=True)
    L = ctypes.CDLL(str(out))
    L.emul_unpack_tile.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    L.emul_codebook_word.restype = ctypes.c_uint32
    L.emul_codebook_word.argtypes = [ctypes.c_int, ctypes.c_uint32]
    L.emul_frag_pos.argtypes = [ctypes.c_void_p]
    return L


@pytest.mark.parametrize("k", range(1, 9))
def test_lane_windows_match_oracle(emul, oracle, k):
    rng = np.random.default_rng(900 + k)
    tiles = rng.integers(0, 65536, size=(40, 16 * k), dtype=np.uint16)
    tiles[0] = 0
    tiles[1] = 0xFFFF
    tiles[2] = 0
    tiles[2, 0] = 0x8001
    tiles[3] = 0
    tiles[3, -1] = 0x8001
    for packed in tiles:
        got = np.empty(256, dtype=np.uint16)
        assert emul.emul_unpack_tile(packed.ctypes.data, k, got.ctypes.data) == 0
        np.testing.assert_array_equal(got, oracle.unpack_trellis_tile(packed, k))


def test_k4_fast_path_matches_oracle(emul, oracle):
    emul.emul_unpack_tile_k4_fast.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    emul.emul_unpack_tile_k4_halves.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    rng = np.random.default_rng(44)
    tiles = rng.integers(0, 65536, size=(200, 64), dtype=np.uint16)
    tiles[0] = 0xFFFF
    tiles[1] = 0
    tiles[1, 0] = 0x8001
    for packed in tiles:
        got = np.empty(256, dtype=np.uint16)
        emul.emul_unpack_tile_k4_fast(packed.ctypes.data, got.ctypes.data)
        np.testing.assert_array_equal(got, oracle.unpack_trellis_tile(packed, 4))
        got[:] = 0
        emul.emul_unpack_tile_k4_halves(packed.ctypes.data, got.ctypes.data)
        np.testing.assert_array_equal(got, oracle.unpack_trellis_tile(packed, 4))


@pytest.mark.parametrize("cb", [0, 1, 2])
def test_codebook_integer_half(emul, oracle, cb):
    table = oracle.codebook_table(cb)
    words = np.array([emul.emul_codebook_word(cb, w) for w in range(65536)], dtype=np.uint32)
    if cb == 2:
        h = (words & 0xFFFF).astype(np.uint16).view(np.float16).astype(np.float64)
        k_inv = np.array([0x1EEE], dtype=np.uint16).view(np.float16)[0].astype(np.float64)
        k_bias = np.array([0xC931], dtype=np.uint16).view(np.float16)[0].astype(np.float64)
        got = (h * k_inv + k_bias).astype(np.float16)
    else:
        lo = (words & 0xFFFF).astype(np.uint16).view(np.float16).astype(np.float64)
        hi = (words >> 16).astype(np.uint16).view(np.float16).astype(np.float64)
        got = (lo + hi).astype(np.float16)
    np.testing.assert_array_equal(got.view(np.uint16), table.view(np.uint16))


def test_fragment_positions(emul, oracle):
    pos = np.empty(256, dtype=np.int32)
    emul.emul_frag_pos(pos.ctypes.data)
    np.testing.assert_array_equal(pos, oracle.tensor_core_perm())
