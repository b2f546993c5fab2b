"""EXL3 quantized linear as a ``torch.nn.Module`` — the drop-in boundary.

Same construction and call contract as the reference's ``EXL3Linear``
(ponyexl3/mlx/exl3_linear.py:56-165): built from an ``EXL3Layer``, called with
``x[..., in]`` (fp16 / bf16 / fp32), returns fp16 ``[..., out]`` with the leading
shape preserved, optional fp16 bias, no autograd, and the packed trellis kept out
of the parameter tree.  Routing by row count replaces the reference's ladder:
rows <= 16 take the streamed GEMV; larger batches take the tensor-core prefill GEMM.
"""

from __future__ import annotations

import numpy as np
import torch

from . import ops
from .layer import EXL3Layer, codebook_mode_from_flags, unpack_signs_or_pass

GEMV_MAX_ROWS = 16


def _to_dev_u16(a: np.ndarray, device: torch.device) -> torch.Tensor:
    a = np.ascontiguousarray(a)
    if a.dtype == np.float16:
        return torch.from_numpy(a.view(np.int16)).to(device).view(torch.float16)
    return torch.from_numpy(a.view(np.int16)).to(device)


class EXL3Linear(torch.nn.Module):
    """One EXL3-quantized linear layer; the trellis stays packed on the device."""

    def __init__(self, layer: EXL3Layer, device: torch.device | str = "cuda"):
        super().__init__()
        layer.validate()
        if layer.in_features % 128 or layer.out_features % 128:
            # the Hadamard rotation is 128-wide (ponyexl3/ref/hadamard.py:67-68)
            raise ValueError("in/out features must be multiples of 128")
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError("EXL3Linear needs a CUDA device: there is no CPU path")
        self.key = layer.key
        self.in_features = layer.in_features
        self.out_features = layer.out_features
        self.k = layer.k
        self.cb = int(codebook_mode_from_flags(mcg=layer.mcg, mul1=layer.mul1))
        suh = unpack_signs_or_pass(layer.suh)
        svh = unpack_signs_or_pass(layer.svh)
        # Plain attributes (not parameters, not buffers): strict state-dict loading of the
        # surrounding model never sees them, as in the reference.
        self._trellis = _to_dev_u16(layer.trellis.astype(np.uint16, copy=False), device)
        self._suh = None if suh is None else _to_dev_u16(suh.astype(np.float16), device)
        self._svh = None if svh is None else _to_dev_u16(svh.astype(np.float16), device)
        self._bias = None if layer.bias is None else _to_dev_u16(layer.bias.astype(np.float16), device)
        self.pdl = False
        self.fast_accum = False

    @classmethod
    def from_device_tensors(cls, *, trellis: torch.Tensor, k: int, cb: int,
                            suh: torch.Tensor | None = None, svh: torch.Tensor | None = None,
                            bias: torch.Tensor | None = None, key: str = "") -> "EXL3Linear":
        """Build the module around tensors that already live on the device (a shard of a
        larger layer, or synthetic weights): trellis (in/16, out/16, 16k) int16, fp16 vectors."""
        if trellis.ndim != 3 or trellis.shape[2] != 16 * k:
            raise ValueError(f"trellis shape {tuple(trellis.shape)} does not fit K={k}")
        if (trellis.shape[0] * 16) % 128 or (trellis.shape[1] * 16) % 128:
            raise ValueError("in/out features must be multiples of 128")
        m = cls.__new__(cls)
        torch.nn.Module.__init__(m)
        m.key = key
        m.in_features, m.out_features = trellis.shape[0] * 16, trellis.shape[1] * 16
        m.k, m.cb = int(k), int(cb)
        m._trellis, m._suh, m._svh, m._bias = trellis.contiguous(), suh, svh, bias
        m.pdl = False
        m.fast_accum = False
        return m

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, k={self.k}, cb={self.cb}"

    @property
    def packed_bytes(self) -> int:
        return self.in_features * self.out_features * self.k // 8

    @torch.no_grad()
    def forward(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """`out`: optional (rows, out_features) fp16 CUDA tensor to write into (unit column stride)."""
        in_shape = x.shape
        if in_shape[-1] != self.in_features:
            raise ValueError(f"expected last dim {self.in_features}, got {in_shape[-1]}")
        x2d = x if x.ndim == 2 else x.reshape(-1, self.in_features)
        rows = x2d.shape[0]
        if rows == 0:
            return torch.empty(in_shape[:-1] + (self.out_features,), dtype=torch.float16,
                               device=x.device)
        if out is not None and (out.shape != (rows, self.out_features) or out.dtype != torch.float16
                                or out.stride(1) != 1):
            raise ValueError("out must be a (rows, out_features) fp16 tensor with unit column stride")
        if rows <= GEMV_MAX_ROWS:
            y = ops.gemv(x2d, self._trellis, self.k, self.cb, self._suh, self._svh, self._bias,
                         pdl=self.pdl, fast_accum=self.fast_accum, out=out)
        else:
            y = ops.gemm(x2d, self._trellis, self.k, self.cb, self._suh, self._svh, self._bias, out=out)
        return y if x.ndim == 2 else y.reshape(in_shape[:-1] + (self.out_features,))
