"""The EXL3 linear layer container, as the reference stores it on disk.

Mirrors ``EXL3Layer`` of the reference (ponyexl3/ref/layer.py:12-44) field for
field so code written against the reference's dataclass works unchanged; arrays
are numpy on the host side and are uploaded once by the module that owns them.
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import IntEnum

import numpy as np


class CodebookMode(IntEnum):
    """ponyexl3/ref/codebook.py:9-12."""
    DEFAULT = 0
    MCG = 1
    MUL1 = 2


def codebook_mode_from_flags(mcg: bool = False, mul1: bool = False) -> CodebookMode:
    """MCG wins over MUL1 (ponyexl3/ref/codebook.py:94-99)."""
    if mcg:
        return CodebookMode.MCG
    if mul1:
        return CodebookMode.MUL1
    return CodebookMode.DEFAULT


def unpack_sign_bitfield(bitfield: np.ndarray) -> np.ndarray:
    """Legacy packed sign words -> +-1 fp16: bit i of word g is channel 16g+i, set
    means -1 (ponyexl3/ref/signs.py:8-19).  Load-time only."""
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


@dataclass
class EXL3Layer:
    """One EXL3-quantized linear layer (ponyexl3/ref/layer.py:12-44)."""

    key: str
    in_features: int
    out_features: int
    k: int
    trellis: np.ndarray  # (in_tiles, out_tiles, 16*k) uint16
    suh: np.ndarray | None = None  # float16 (in,) or packed int16 (in//16,)
    svh: np.ndarray | None = None
    bias: np.ndarray | None = None
    mcg: bool = False
    mul1: bool = False

    @property
    def codebook_mode(self) -> int:
        return int(codebook_mode_from_flags(mcg=self.mcg, mul1=self.mul1))

    @property
    def packed_tile_size(self) -> int:
        return 256 * self.k // 16

    def validate(self) -> None:
        in_tiles = self.in_features // 16
        out_tiles = self.out_features // 16
        if self.in_features % 16 != 0 or self.out_features % 16 != 0:
            raise ValueError("in/out features must be multiples of 16")
        if not 1 <= self.k <= 8:
            raise ValueError(f"K must be in [1, 8], got {self.k}")
        if self.trellis.shape != (in_tiles, out_tiles, self.packed_tile_size):
            raise ValueError(
                f"trellis shape {self.trellis.shape} != "
                f"expected {(in_tiles, out_tiles, self.packed_tile_size)}")
