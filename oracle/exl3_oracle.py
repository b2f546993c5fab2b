"""numpy front end of the CPU oracle (``exl3_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Only the test suite, the smoke check and the benchmark's CPU-baseline legs may
import this module; the product package never does.  Function names and
argument meaning follow the reference's ``ponyexl3.ref`` package so that parity
tests read like the reference's own (each docstring names the function it
mirrors, as path-in-reference:lines).

Parity is pinned against vectors made by the reference itself
(``tests/golden/make_golden.py``).
"""

from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libexl3_oracle.so"
_lib: ctypes.CDLL | None = None

CB_3INST, CB_MCG, CB_MUL1 = 0, 1, 2


def build(force: bool = False) -> Path:
    """Compile ``exl3_oracle.c`` with the Makefile beside it (gcc, OpenMP)."""
    src = _HERE / "exl3_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-s", "clean", "all"], check=True,
                       stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(_LIB_PATH))
        i64, p, i32 = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
        L.exl3o_decode_codeword.restype = ctypes.c_uint16
        L.exl3o_decode_codeword.argtypes = [ctypes.c_uint32, i32]
        L.exl3o_codebook_table.argtypes = [i32, p]
        L.exl3o_unpack_tile.argtypes = [p, i32, p]
        L.exl3o_pack_tile.argtypes = [p, i32, p]
        L.exl3o_tile_perm.argtypes = [p]
        L.exl3o_unpack.argtypes = [p, i64, i32, p]
        L.exl3o_decode_trellis.argtypes = [p, i64, i64, i32, i32, i64, i64, p, i64]
        L.exl3o_had128.argtypes = [p, i64, i64, p, p, p]
        L.exl3o_forward_w.argtypes = [p, i64, i64, i64, p, p, p, p, p]
        L.exl3o_forward.argtypes = [p, i64, p, i64, i64, i32, i32, p, p, p, p]
        L.exl3o_half_to_float.argtypes = [p, p, i64]
        L.exl3o_double_to_half.argtypes = [p, p, i64]
        L.exl3o_quantize_tile.argtypes = [p, i32, i32, i32, p]
        L.exl3o_num_threads.restype = i32
        L.exl3o_set_threads.argtypes = [i32]
        _lib = L
    return _lib


def _ptr(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _u16(a: np.ndarray | None) -> np.ndarray | None:
    """fp16/uint16/int16 array -> contiguous uint16 bit view."""
    if a is None:
        return None
    a = np.ascontiguousarray(a)
    if a.dtype == np.float16:
        return a.view(np.uint16)
    if a.dtype in (np.uint16, np.int16):
        return a.view(np.uint16)
    return np.ascontiguousarray(a.astype(np.float16)).view(np.uint16)


def codebook_mode(mcg: bool = False, mul1: bool = False) -> int:
    """ponyexl3/ref/codebook.py:94-99 (codebook_mode_from_flags): MCG wins over MUL1."""
    return CB_MCG if mcg else (CB_MUL1 if mul1 else CB_3INST)


def decode_3inst(codeword: int, cb: int) -> np.float16:
    """ponyexl3/ref/codebook.py:66-91."""
    bits = lib().exl3o_decode_codeword(int(codeword) & 0xFFFF, int(cb))
    return np.array([bits], dtype=np.uint16).view(np.float16)[0]


def codebook_table(cb: int) -> np.ndarray:
    """All 65,536 codewords decoded, as float16."""
    t = np.empty(65536, dtype=np.uint16)
    lib().exl3o_codebook_table(int(cb), _ptr(t))
    return t.view(np.float16)


def unpack_trellis_tile(packed: np.ndarray, k: int) -> np.ndarray:
    """ponyexl3/ref/trellis.py:105-141.  (16K,) uint16 -> (256,) uint16 codewords."""
    packed = np.ascontiguousarray(packed, dtype=np.uint16)
    if packed.shape != (16 * k,):
        raise ValueError(f"expected packed shape ({16 * k},), got {packed.shape}")
    out = np.empty(256, dtype=np.uint16)
    if lib().exl3o_unpack_tile(_ptr(packed), k, _ptr(out)) != 0:
        raise ValueError(f"K must be in [1, 8], got {k}")
    return out


def pack_trellis_tile(encoded: np.ndarray, k: int) -> np.ndarray:
    """ponyexl3/ref/trellis.py:12-50.  (256,) uint16 (low K bits used) -> (16K,) uint16."""
    encoded = np.ascontiguousarray(encoded, dtype=np.uint16)
    if encoded.shape != (256,):
        raise ValueError(f"expected encoded shape (256,), got {encoded.shape}")
    if not 1 <= k <= 8:
        raise ValueError(f"K must be in [1, 8], got {k}")
    out = np.empty(16 * k, dtype=np.uint16)
    lib().exl3o_pack_tile(_ptr(encoded), k, _ptr(out))
    return out


def pack_trellis(encoded: np.ndarray, k: int) -> np.ndarray:
    """ponyexl3/ref/trellis.py:144-150.  (tiles_k, tiles_n, 256) -> (tiles_k, tiles_n, 16K)."""
    if encoded.ndim != 3 or encoded.shape[-1] != 256:
        raise ValueError(f"expected shape (tiles_k, tiles_n, 256), got {encoded.shape}")
    out = np.empty(encoded.shape[:2] + (16 * k,), dtype=np.uint16)
    for i in range(encoded.shape[0]):
        for j in range(encoded.shape[1]):
            out[i, j] = pack_trellis_tile(encoded[i, j], k)
    return out


def unpack_trellis(packed: np.ndarray, k: int) -> np.ndarray:
    """ponyexl3/ref/trellis.py:205-214.  (tiles_k, tiles_n, 16K) -> (tiles_k, tiles_n, 256)."""
    if packed.ndim != 3:
        raise ValueError(f"expected 3D packed trellis, got {packed.shape}")
    if packed.shape[-1] != 16 * k:
        raise ValueError(f"expected last dim {16 * k}, got {packed.shape[-1]}")
    packed = np.ascontiguousarray(packed, dtype=np.uint16)
    out = np.empty(packed.shape[:2] + (256,), dtype=np.uint16)
    lib().exl3o_unpack(_ptr(packed), packed.shape[0] * packed.shape[1], k, _ptr(out))
    return out


def quantize_tile(w: np.ndarray, k: int, cb: int = 0, max_pins: int = 4) -> tuple[np.ndarray, np.ndarray]:
    """ponyexl3/convert/reference_search.py:60-87 (quantize_tile_reference): exact Viterbi search of
    one tile.  w (256,) float32 in codeword order -> (states (256,) uint16, decoded (256,) float32)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    if w.shape != (256,):
        raise ValueError(f"expected w shape (256,), got {w.shape}")
    states = np.empty(256, dtype=np.uint16)
    if lib().exl3o_quantize_tile(_ptr(w), int(k), int(cb), int(max_pins), _ptr(states)) != 0:
        raise ValueError("bad K, codebook or max_pins")
    return states, codebook_table(cb)[states].astype(np.float32)


def tensor_core_perm() -> np.ndarray:
    """ponyexl3/ref/perm.py:8-26: tile position row*16+col of codeword index i."""
    p = np.empty(256, dtype=np.int32)
    lib().exl3o_tile_perm(_ptr(p))
    return p


def decode_packed_trellis(trellis: np.ndarray, k: int, cb: int, *, n_offset: int = 0,
                          n_count: int | None = None) -> np.ndarray:
    """ponyexl3/ref/decode.py:32-81: inner W (in, n_count) float16."""
    if trellis.ndim != 3:
        raise ValueError("trellis must be 3D")
    t_in, t_out, ps = trellis.shape
    if ps != 16 * k:
        raise ValueError(f"packed size {ps} != expected {16 * k} for K={k}")
    if n_offset % 128 != 0:
        raise ValueError("n_offset must be divisible by 128")
    n_count = t_out * 16 - n_offset if n_count is None else n_count
    if n_offset + n_count > t_out * 16 or n_count % 16:
        raise ValueError("slice exceeds output features")
    trellis = np.ascontiguousarray(trellis, dtype=np.uint16)
    w = np.empty((t_in * 16, n_count), dtype=np.uint16)
    rc = lib().exl3o_decode_trellis(_ptr(trellis), t_in, t_out, k, int(cb), n_offset // 16,
                                    n_count // 16, _ptr(w), n_count)
    if rc != 0:
        raise ValueError(f"decode failed ({rc})")
    return w.view(np.float16)


def had_r_128(x: np.ndarray, *, pre_scale: np.ndarray | None = None,
              post_scale: np.ndarray | None = None) -> np.ndarray:
    """ponyexl3/ref/hadamard.py:50-80, float32 in and out."""
    if x.ndim != 2:
        raise ValueError("had_r_128 expects 2D input (rows, features)")
    if x.shape[1] % 128 != 0:
        raise ValueError(f"feature dim {x.shape[1]} not divisible by 128")
    xf = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(xf)
    pre, post = _u16(pre_scale), _u16(post_scale)
    lib().exl3o_had128(_ptr(xf), xf.shape[0], xf.shape[1], _ptr(pre), _ptr(post), _ptr(y))
    return y


def unpack_sign_bitfield(bitfield: np.ndarray) -> np.ndarray:
    """ponyexl3/ref/signs.py:8-19: bit i of word g -> channel 16g+i, set means -1."""
    bf = np.asarray(bitfield).astype(np.uint16).reshape(-1, 1)
    bits = (bf >> np.arange(16, dtype=np.uint16).reshape(1, 16)) & 1
    return np.where(bits != 0, -1.0, 1.0).astype(np.float16).reshape(-1)


def unpack_signs_or_pass(values: np.ndarray | None) -> np.ndarray | None:
    """ponyexl3/ref/signs.py:22-27."""
    if values is None:
        return None
    if values.dtype in (np.float16, np.float32):
        return values.astype(np.float16, copy=False)
    return unpack_sign_bitfield(values)


def linear_forward(x: np.ndarray, trellis: np.ndarray, k: int, cb: int,
                   suh: np.ndarray | None, svh: np.ndarray | None,
                   bias: np.ndarray | None = None, w: np.ndarray | None = None) -> np.ndarray:
    """ponyexl3/ref/forward.py:14-49 (linear_forward_reconstruct); fp16 in, fp16 out.

    ``w`` may carry an already decoded inner matrix (in, out) to skip the decode.
    """
    t_in, t_out, _ = trellis.shape
    x = np.asarray(x)
    lead = x.shape[:-1]
    x2 = np.ascontiguousarray(x.reshape(-1, t_in * 16).astype(np.float16))
    rows = x2.shape[0]
    suh, svh = unpack_signs_or_pass(suh), unpack_signs_or_pass(svh)
    y = np.empty((rows, t_out * 16), dtype=np.uint16)
    bias16 = _u16(bias)
    if w is None:
        tr = np.ascontiguousarray(trellis, dtype=np.uint16)
        rc = lib().exl3o_forward(_ptr(_u16(x2)), rows, _ptr(tr), t_in, t_out, k, int(cb),
                                 _ptr(_u16(suh)), _ptr(_u16(svh)), _ptr(bias16), _ptr(y))
    else:
        rc = lib().exl3o_forward_w(_ptr(_u16(x2)), rows, t_in * 16, t_out * 16, _ptr(_u16(w)),
                                   _ptr(_u16(suh)), _ptr(_u16(svh)), _ptr(bias16), _ptr(y))
    if rc != 0:
        raise ValueError(f"forward failed ({rc})")
    return y.view(np.float16).reshape(lead + (t_out * 16,))


def glu(g: np.ndarray, u: np.ndarray, activation: str = "silu") -> np.ndarray:
    """Gate activation of the stacked experts, float32 math then fp16
    (ponyexl3/mlx/exl3_moe.py:62-75): silu(g)*u or tanh-gelu(g)*u."""
    g = g.astype(np.float32)
    u = u.astype(np.float32)
    if activation == "gelu":
        h = 0.5 * g * (1.0 + np.tanh(0.797884560803 * (g + 0.044715 * g * g * g))) * u
    elif activation == "silu":
        h = (g / (1.0 + np.exp(-g))) * u
    else:
        raise ValueError(f"unsupported MoE activation {activation!r}")
    return h.astype(np.float16)


def switch_glu(x: np.ndarray, indices: np.ndarray, *, gu_trellis: np.ndarray, gu_suh: np.ndarray,
               gu_svh: np.ndarray, dn_trellis: np.ndarray, dn_suh: np.ndarray, dn_svh: np.ndarray,
               k: int, cb: int, activation: str = "silu") -> np.ndarray:
    """Stacked-expert SwitchGLU, composed from the linear forward per (row, slot)
    (ponyexl3/mlx/exl3_moe.py:634-683, the unfused decode path ``_decode``):
    gate and up are two EXL3 linears D->H with their own suh rows and the halves
    of gu_svh, h = fp16(glu(g, u)), down is an EXL3 linear H->D.

    x (R, D) fp16; indices (R, kk) -> (R, kk, D) fp16, un-weighted expert outputs.
    gu_trellis (D/16, E*2*H/16, 16K) holds all gates then all ups; dn_trellis
    (H/16, E*D/16, 16K).
    """
    E, _, D = gu_suh.shape
    H = dn_suh.shape[1]
    gt, dt = H // 16, D // 16
    R, kk = indices.shape
    out = np.empty((R, kk, D), dtype=np.float16)
    cache: dict[int, tuple[np.ndarray, np.ndarray, np.ndarray]] = {}
    for r in range(R):
        for s in range(kk):
            e = int(indices[r, s])
            if e not in cache:
                wg = decode_packed_trellis(gu_trellis[:, e * gt:(e + 1) * gt], k, cb)
                wu = decode_packed_trellis(gu_trellis[:, (E + e) * gt:(E + e + 1) * gt], k, cb)
                wd = decode_packed_trellis(dn_trellis[:, e * dt:(e + 1) * dt], k, cb)
                cache[e] = (wg, wu, wd)
            wg, wu, wd = cache[e]
            xr = x[r:r + 1]
            g = linear_forward(xr, gu_trellis[:, e * gt:(e + 1) * gt], k, cb, gu_suh[e, 0],
                               gu_svh[e, :H], w=wg)
            u = linear_forward(xr, gu_trellis[:, (E + e) * gt:(E + e + 1) * gt], k, cb,
                               gu_suh[e, 1], gu_svh[e, H:], w=wu)
            h = glu(g, u, activation)
            out[r, s] = linear_forward(h, dn_trellis[:, e * dt:(e + 1) * dt], k, cb, dn_suh[e],
                                       dn_svh[e], w=wd)[0]
    return out


def num_threads() -> int:
    return int(lib().exl3o_num_threads())


def set_threads(n: int) -> None:
    lib().exl3o_set_threads(int(n))


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1
