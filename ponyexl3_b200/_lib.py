"""ctypes binding of ``libexl3b200.so`` (the C ABI declared in ``include/exl3_b200.h``).

There is no fallback: if the library is missing or a call fails, an exception is
raised.  ``check(rc)`` maps the negative EXL3_E* codes to Python exceptions the way
the reference's host code raises them (``ValueError`` for shape / K / dtype
problems, ``RuntimeError`` for CUDA failures).
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_uint, c_void_p
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "lib" / "libexl3b200.so"

DT_F16, DT_BF16, DT_F32 = 0, 1, 2
FLAG_PDL = 1
FLAG_FAST_ACCUM = 2
FLAG_GLU_SILU = 4
FLAG_GLU_GELU = 8

E_CUDA = -9
E_UNSUPPORTED = -11
_VALUE_ERRORS = {-1, -2, -3, -4, -5, -6, -7, -8, -10, -11}

_PROTOTYPES = {
    "exl3_version": (c_int, []),
    "exl3_error_string": (c_char_p, [c_int]),
    "exl3_last_cuda_error": (c_char_p, []),
    "exl3_unpack": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p]),
    "exl3_decode": (c_int, [c_void_p, c_int64, c_int64, c_int, c_int, c_int64, c_int64, c_void_p,
                            c_int64, c_void_p]),
    "exl3_codebook_table": (c_int, [c_int, c_void_p, c_void_p]),
    "exl3_hadamard128": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p,
                                 c_void_p, c_void_p]),
    "exl3_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "exl3_workspace_init": (c_int, [c_void_p, c_size_t, c_void_p]),
    "exl3_workspace_status": (c_int, [c_void_p, ctypes.POINTER(c_int), c_void_p]),
    "exl3_gemv": (c_int, [c_void_p, c_int, c_int, c_int64, c_void_p, c_int64, c_int64, c_int, c_int,
                          c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_size_t,
                          c_uint, c_void_p]),
    "exl3_gemv_blocks": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_int64, c_int64, c_int, c_int, c_void_p, c_int64, c_int,
                                 c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_size_t,
                                 c_uint, c_void_p]),
    "exl3_gemv_blocks_counted": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_int64, c_int64, c_int, c_int, c_void_p, c_int64, c_void_p,
                                         c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p,
                                         c_size_t, c_uint, c_void_p]),
    "exl3_gemm_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "exl3_gemm": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int, c_int,
                          c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_size_t,
                          c_uint, c_void_p]),
    "exl3_gemm_tiles": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_int64, c_int64, c_int, c_int, c_void_p, c_int64,
                                c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_size_t, c_uint, c_void_p]),
    "exl3_gemm_tiles_peers": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_int64, c_int64, c_int, c_int, c_void_p, c_int64, c_void_p,
                                      c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_void_p,
                                      c_size_t, c_uint, c_void_p]),
    "exl3_gemv_noalloc": (c_int, [c_void_p, c_int, c_int, c_int64, c_void_p, c_int64, c_int64, c_int,
                                  c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_uint,
                                  c_void_p]),
    "exl3_gemv_noalloc_status": (c_int, [ctypes.POINTER(c_int), c_void_p]),
    "exl3_add_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64,
                                 c_int64, ctypes.c_float, c_uint, c_void_p]),
    "exl3_rope_append": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                 c_int, c_int, c_int64, c_int, c_uint, c_void_p]),
    "exl3_attn_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int64]),
    "exl3_attn_decode": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int,
                                 c_void_p, c_size_t, c_uint, c_void_p]),
    "exl3_swiglu": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int64, c_uint, c_void_p]),
    "exl3_gemv_peers": (c_int, [c_void_p, c_int, c_int, c_int64, c_void_p, c_int64, c_int64, c_int, c_int,
                                c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64,
                                c_void_p, c_size_t, c_uint, c_void_p]),
    "exl3_gemv_peers_after": (c_int, [c_void_p, c_int, c_int, c_int64, c_void_p, c_int64, c_int64, c_int, c_int,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64,
                                      c_void_p, c_uint, c_void_p, c_size_t, c_uint, c_void_p]),
    "exl3_peer_allgather": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p, c_int, c_int64,
                                    c_int64, c_uint, c_void_p]),
    "exl3_peer_wait": (c_int, [c_void_p, c_uint, c_void_p, c_uint, c_void_p]),
    "exl3_tune_gemv": (None, [c_int, c_int]),
    "exl3_tune_gemm": (None, [c_int]),
    "exl3_tune_gemm_pairs": (None, [c_int]),
    "exl3_moe_prefill_tables": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int64, c_void_p, c_void_p,
                                        c_void_p, c_void_p, c_void_p, c_void_p, c_uint, c_void_p]),
    "exl3_moe_decode_tables": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int64, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_void_p, c_uint, c_void_p]),
    "exl3_moe_prefill_tables_range": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int64, c_int64,
                                              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_uint, c_void_p]),
    "exl3_encode_workspace_bytes": (c_size_t, [c_int64]),
    "exl3_encode_tiles": (c_int, [c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_size_t,
                                  c_void_p]),
    "exl3_moe_decode_tables_range": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int64, c_int64,
                                             c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_uint, c_void_p]),
}

_lib: ctypes.CDLL | None = None


def use_library(path: Path) -> None:
    """Bind another build of the library (the timeline build of ``ponyexl3_b200.profiling``).
    Must be called before the first ``load()``."""
    global LIB_PATH
    if _lib is not None:
        raise RuntimeError("the library is already loaded")
    LIB_PATH = Path(path)


def load() -> ctypes.CDLL:
    """The loaded library; raises if it has not been built (``python -m ponyexl3_b200.build``)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m ponyexl3_b200.build` "
                "(there is no CPU or PyTorch fallback for the EXL3 path)")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in _PROTOTYPES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def prototypes() -> dict:
    return dict(_PROTOTYPES)


def check(rc: int, what: str = "") -> None:
    if rc == 0:
        return
    lib = load()
    msg = lib.exl3_error_string(rc).decode()
    if rc == E_CUDA:
        raise RuntimeError(f"{what}: {msg}: {lib.exl3_last_cuda_error().decode()}")
    if rc in _VALUE_ERRORS:
        raise ValueError(f"{what}: {msg} (code {rc})")
    raise RuntimeError(f"{what}: {msg} (code {rc})")
