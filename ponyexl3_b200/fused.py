"""Fused EXL3 sibling groups — several same-input, same-K linears in one launch.

Mirrors ``FusedEXL3Group`` / ``FusedEXL3Sibling`` of the reference
(ponyexl3/mlx/exl3_fused.py:80-233): the members' trellises are concatenated along the
out-tile axis, their ``suh`` rows stacked (each member rotates the input with its own
signs), their ``svh`` concatenated (member widths are multiples of 128, so an output
rotation block never straddles two members), and ``forward_all`` returns one output per
member.  On the B200 the group is one rotation launch plus one streamed GEMV over a block
table (``exl3_gemv_blocks``) for up to 16 rows, and per-member tensor-core GEMMs above that.
"""

from __future__ import annotations

import numpy as np
import torch

from . import ops
from .layer import EXL3Layer, codebook_mode_from_flags, unpack_signs_or_pass
from .linear import GEMV_MAX_ROWS, _to_dev_u16


def fusable(layers: list[EXL3Layer]) -> bool:
    """Same rule as the reference (ponyexl3/mlx/exl3_fused.py:80-90)."""
    first = layers[0]
    return (
        len(layers) >= 2
        and all(l.in_features == first.in_features for l in layers)
        and all(l.k == first.k for l in layers)
        and all((l.mcg, l.mul1) == (first.mcg, first.mul1) for l in layers)
        and all(l.out_features % 128 == 0 for l in layers)
        and all(l.suh is not None and l.svh is not None for l in layers)
        and all(l.bias is None for l in layers)
    )


class FusedEXL3Group(torch.nn.Module):
    """Owner of the concatenated trellis + stacked signs for sibling linears."""

    def __init__(self, layers: list[EXL3Layer], device: torch.device | str = "cuda"):
        super().__init__()
        if not fusable(layers):
            raise ValueError("layers not fusable: " + ", ".join(l.key for l in layers))
        for l in layers:
            l.validate()
        if layers[0].in_features % 128:
            raise ValueError("in_features must be a multiple of 128")
        device = torch.device(device)
        self._keys = [l.key for l in layers]
        self.k = layers[0].k
        self.cb = int(codebook_mode_from_flags(mcg=layers[0].mcg, mul1=layers[0].mul1))
        self.in_features = layers[0].in_features
        self._out_features = [l.out_features for l in layers]
        self._trellis = _to_dev_u16(
            np.concatenate([l.trellis for l in layers], axis=1).astype(np.uint16), device)
        self._suh_stack = _to_dev_u16(
            np.stack([unpack_signs_or_pass(l.suh) for l in layers]).astype(np.float16), device)
        self._svh_cat = _to_dev_u16(
            np.concatenate([unpack_signs_or_pass(l.svh) for l in layers]).astype(np.float16), device)
        # member index of every 128-column block
        self._block_sub = np.repeat(np.arange(len(layers)), [n // 128 for n in self._out_features])
        self._offsets = np.concatenate([[0], np.cumsum(self._out_features)]).astype(np.int64)
        self._tables: dict[int, tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}
        self._cache_x: torch.Tensor | None = None
        self._cache_out: tuple[torch.Tensor, ...] | None = None
        self.pdl = False

    @classmethod
    def from_device_tensors(cls, *, trellis: torch.Tensor, k: int, cb: int, suh_stack: torch.Tensor,
                            svh_cat: torch.Tensor, out_features: list[int],
                            keys: list[str] | None = None) -> "FusedEXL3Group":
        """Build the group around tensors already on the device (a shard, or synthetic weights):
        trellis (in/16, sum(out)/16, 16k) int16 with the members side by side, suh_stack
        (members, in) fp16, svh_cat (sum(out),) fp16."""
        total = sum(out_features)
        if trellis.ndim != 3 or trellis.shape[2] != 16 * k or trellis.shape[1] * 16 != total:
            raise ValueError(f"trellis shape {tuple(trellis.shape)} does not fit K={k}, out={total}")
        if (trellis.shape[0] * 16) % 128 or any(n % 128 for n in out_features):
            raise ValueError("in features and member widths must be multiples of 128")
        if tuple(suh_stack.shape) != (len(out_features), trellis.shape[0] * 16) or svh_cat.numel() != total:
            raise ValueError("suh_stack / svh_cat do not match the members")
        g = cls.__new__(cls)
        torch.nn.Module.__init__(g)
        g._keys = list(keys) if keys else [f"member{i}" for i in range(len(out_features))]
        g.k, g.cb = int(k), int(cb)
        g.in_features = trellis.shape[0] * 16
        g._out_features = [int(n) for n in out_features]
        g._trellis, g._suh_stack, g._svh_cat = trellis.contiguous(), suh_stack.contiguous(), svh_cat
        g._block_sub = np.repeat(np.arange(len(out_features)), [n // 128 for n in out_features])
        g._offsets = np.concatenate([[0], np.cumsum(g._out_features)]).astype(np.int64)
        g._tables = {}
        g._cache_x = g._cache_out = None
        g.pdl = False
        return g

    def extra_repr(self) -> str:
        return f"members={self._keys}, k={self.k}"

    @property
    def packed_bytes(self) -> int:
        return self.in_features * int(self._offsets[-1]) * self.k // 8

    def _table(self, rows: int, device: torch.device):
        """Block table and rotation indices for `rows` activation rows (cached per row count):
        rotated row sub*rows + r = had(x[r] * suh[sub])."""
        t = self._tables.get(rows)
        if t is None:
            nb = len(self._block_sub)
            b = np.arange(nb, dtype=np.int32)
            blocks = np.stack([b, self._block_sub.astype(np.int32) * rows, b * 128, b * 128], axis=1)
            n_sub = len(self._out_features)
            row_src = np.tile(np.arange(rows, dtype=np.int32), n_sub)
            suh_row = np.repeat(np.arange(n_sub, dtype=np.int32), rows)
            t = (torch.from_numpy(np.ascontiguousarray(blocks)).to(device),
                 torch.from_numpy(row_src).to(device), torch.from_numpy(suh_row).to(device))
            self._tables[rows] = t
        return t

    @torch.no_grad()
    def forward_packed(self, x2d: torch.Tensor) -> torch.Tensor:
        """All members side by side, (rows, sum(out)) fp16, for 1..16 rows — one buffer a
        following kernel can take whole (q|k|v for the rotary step, gate|up for SwiGLU)."""
        rows = x2d.shape[0]
        if not 1 <= rows <= GEMV_MAX_ROWS:
            raise ValueError("forward_packed serves 1..16 rows")
        blocks, row_src, suh_row = self._table(rows, x2d.device)
        y = torch.empty((rows, int(self._offsets[-1])), dtype=torch.float16, device=x2d.device)
        ops.gemv_blocks(x2d, xh_rows=rows * len(self._out_features), row_src=row_src,
                        suh=self._suh_stack, suh_row=suh_row, trellis=self._trellis, k=self.k,
                        cb=self.cb, blocks=blocks, rows=rows, svh=self._svh_cat, bias=None, y=y,
                        pdl=self.pdl)
        return y

    @torch.no_grad()
    def forward_all(self, x: torch.Tensor) -> tuple[torch.Tensor, ...]:
        in_shape = x.shape
        if in_shape[-1] != self.in_features:
            raise ValueError(f"expected last dim {self.in_features}, got {in_shape[-1]}")
        x2d = x.reshape(-1, self.in_features)
        rows = x2d.shape[0]
        total = int(self._offsets[-1])
        if rows == 0:
            return tuple(torch.empty(in_shape[:-1] + (n,), dtype=torch.float16, device=x.device)
                         for n in self._out_features)
        if rows <= GEMV_MAX_ROWS:
            blocks, row_src, suh_row = self._table(rows, x.device)
            y = torch.empty((rows, total), dtype=torch.float16, device=x.device)
            ops.gemv_blocks(x2d, xh_rows=rows * len(self._out_features), row_src=row_src,
                            suh=self._suh_stack, suh_row=suh_row, trellis=self._trellis, k=self.k,
                            cb=self.cb, blocks=blocks, rows=rows, svh=self._svh_cat, bias=None, y=y,
                            pdl=self.pdl)
            outs = [y[:, int(a):int(b)] for a, b in zip(self._offsets[:-1], self._offsets[1:])]
        else:
            # prefill: one tensor-core GEMM per member on its out-tile range of the shared trellis
            outs = []
            for i, n in enumerate(self._out_features):
                t0 = int(self._offsets[i]) // 16
                tr = self._trellis[:, t0:t0 + n // 16].contiguous()
                outs.append(ops.gemm(x2d, tr, self.k, self.cb, self._suh_stack[i],
                                     self._svh_cat[int(self._offsets[i]):int(self._offsets[i + 1])], None))
        return tuple(o.reshape(in_shape[:-1] + (n,)) for o, n in zip(outs, self._out_features))

    def cached(self, x: torch.Tensor) -> tuple[torch.Tensor, ...]:
        """Single-slot cache keyed on input identity (ponyexl3/mlx/exl3_fused.py:204-208)."""
        if self._cache_out is None or self._cache_x is not x:
            self._cache_out = self.forward_all(x)
            self._cache_x = x
        return self._cache_out

    def sibling(self, idx: int) -> "FusedEXL3Sibling":
        return FusedEXL3Sibling(self, idx)


class FusedEXL3Sibling(torch.nn.Module):
    """Drop-in replacement for one member linear; delegates to the group."""

    def __init__(self, group: FusedEXL3Group, idx: int):
        super().__init__()
        self.__dict__["_group"] = group      # not a sub-module: the group owns the weights
        self._idx = idx
        self.in_features = group.in_features
        self.out_features = group._out_features[idx]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self._group.cached(x)[self._idx]
