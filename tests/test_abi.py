"""The C ABI library loads and exports every symbol the headers under ``include/`` declare,
the Python binding declares the same set, and host-side validation rejects bad
arguments before anything touches a GPU (no compute calls here)."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _declared() -> list[str]:
    text = "\n".join(p.read_text() for p in sorted((ROOT / "include").glob("*.h")))
    return re.findall(r"^EXL3_API\s+[\w\s\*]+?\b(exl3_\w+)\s*\(", text, flags=re.M)


@pytest.fixture(scope="module")
def lib():
    from ponyexl3_b200 import build, _lib

    build.build()
    return _lib.load()


def test_every_declared_symbol_is_exported_and_bound(lib):
    from ponyexl3_b200 import _lib

    names = _declared()
    assert len(names) >= 11
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert set(names) == set(_lib.prototypes()), "header and ctypes binding disagree"


def test_header_cites_the_reference_for_each_entry_point():
    text = (ROOT / "include" / "exl3_b200.h").read_text()
    assert text.count("ponyexl3/") >= 8


def test_version_and_error_strings(lib):
    assert lib.exl3_version() == 100
    for code in range(0, -12, -1):
        assert lib.exl3_error_string(code)
    assert b"unknown" in lib.exl3_error_string(-99)


def test_host_side_validation_needs_no_gpu(lib):
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    p = (p + 255) & ~255  # aligned fake pointers: validation must fail before any launch
    assert lib.exl3_unpack(None, 1, 4, p, None) == -1
    assert lib.exl3_unpack(p, 1, 9, p, None) == -2
    assert lib.exl3_decode(p, 1, 1, 4, 3, 0, 1, p, 16, None) == -3
    assert lib.exl3_decode(p, 1, 1, 4, 0, 1, 1, p, 16, None) == -10
    assert lib.exl3_hadamard128(p, 0, 1, 100, 100, None, None, p, None) == -4
    assert lib.exl3_hadamard128(p, 7, 1, 128, 128, None, None, p, None) == -8
    assert lib.exl3_workspace_bytes(16, 17408) > lib.exl3_workspace_bytes(1, 4096) >= 256 + 4096 * 4
    gemv = lambda **kw: lib.exl3_gemv(
        kw.get("x", p), kw.get("dt", 0), kw.get("rows", 1), kw.get("xs", 128), kw.get("tr", p),
        kw.get("t_in", 8), kw.get("t_out", 8), kw.get("k", 4), kw.get("cb", 0), None, None, None,
        kw.get("y", p), kw.get("ys", 128), kw.get("ws", p), kw.get("wsb", 1 << 30), 0, None)
    assert gemv(x=None) == -1
    assert gemv(k=0) == -2
    assert gemv(cb=5) == -3
    assert gemv(t_in=7) == -4
    assert gemv(rows=17) == -5
    assert gemv(rows=0) == -5
    assert gemv(x=p + 2) == -6
    assert gemv(ws=None) == -7
    assert gemv(wsb=16) == -7
    assert gemv(dt=9) == -8
    # the expert-parallel entry points: ranges, counts and peer tables are checked on the host
    tabs = lambda f, lo, hi, counts: f(p, 8, 16, 4, 8, lo, hi, 256, 128, p, p, p, p, p, counts, 0, None)
    assert tabs(lib.exl3_moe_decode_tables_range, 0, 4, None) == -1
    assert tabs(lib.exl3_moe_decode_tables_range, 4, 4, p) == -10
    assert tabs(lib.exl3_moe_decode_tables_range, 0, 9, p) == -10
    assert lib.exl3_moe_decode_tables_range(p, 8, 4096, 4, 8, 0, 4, 256, 128, p, p, p, p, p, p, 0, None) == -10
    ptabs = lambda lo, hi, counts: lib.exl3_moe_prefill_tables_range(p, 8, 512, 4, 8, lo, hi, 256, 128, p, p, p, p, p, p,
                                                                    counts, 0, None)
    assert ptabs(0, 4, None) == -1
    assert ptabs(5, 4, p) == -10
    blocks = lambda cnt: lib.exl3_gemv_blocks_counted(p, 0, 128, 1, None, None, None, p, 8, 8, 4, 0, p, 1, cnt, 1, None,
                                                      None, p, 128, 0, p, 1 << 30, 0, None)
    assert blocks(None) == -1
    assert blocks(p + 2) == -6
    u64 = (ctypes.c_uint64 * 2)(p, p)
    tiles = lambda **kw: lib.exl3_gemm_tiles_peers(p, 0, 128, 256, None, None, None, None, p, 8, 8, 4, 0, p, 1, None,
                                                   kw.get("y", p), 128, kw.get("map", p), kw.get("yp", u64),
                                                   kw.get("cp", u64), kw.get("n", 2), kw.get("rpp", 128), p, 1 << 30, 0,
                                                   None)
    assert tiles(n=9) == -10
    assert tiles(map=None) == -1
    assert tiles(yp=None) == -1
    assert tiles(rpp=0) == -1


def test_layer_container_mirrors_reference_validation():
    import numpy as np
    from ponyexl3_b200 import EXL3Layer

    tr = np.zeros((8, 8, 64), dtype=np.uint16)
    EXL3Layer("a", 128, 128, 4, tr).validate()
    with pytest.raises(ValueError):
        EXL3Layer("a", 128, 128, 3, tr).validate()
    with pytest.raises(ValueError):
        EXL3Layer("a", 120, 128, 4, tr).validate()
    assert EXL3Layer("a", 128, 128, 4, tr, mcg=True, mul1=True).codebook_mode == 1
    assert EXL3Layer("a", 128, 128, 4, tr, mul1=True).codebook_mode == 2
    assert EXL3Layer("a", 128, 128, 4, tr).packed_tile_size == 64


def test_ops_refuse_cpu_tensors():
    import torch
    from ponyexl3_b200 import ops

    with pytest.raises(RuntimeError):
        ops.unpack_trellis(torch.zeros((1, 1, 64), dtype=torch.int16), 4)
    with pytest.raises(RuntimeError):
        ops.had_r_128(torch.zeros((1, 128)))
