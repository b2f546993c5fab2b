"""Dense gated MLP as one module: gate|up in one launch, the GLU folded into the down launch.

Mirrors ``EXL3MLPMonolith`` of the reference (ponyexl3/mlx/exl3_mlp_monolith.py:37-119): a
drop-in for a model's ``gate_proj`` / ``up_proj`` / ``down_proj`` triple built from the fused
gate/up sibling group and the down linear, with the same numerics as running the three linears
and the activation one after the other (``h`` is rounded to fp16 between the GLU and the down
projection, as there).

Up to 16 rows the call is two streamed-GEMV launches: the sibling group writes ``[gate | up]``,
and the down projection reads that buffer as it is, applying ``act(gate) * up`` while it loads
its activations (EXL3_FLAG_GLU_*), so there is no activation kernel and no ``h`` buffer in
between.  More rows go through the tensor-core GEMM per member, with the GLU as a separate
kernel.
"""

from __future__ import annotations

import torch

from . import ops
from .fused import FusedEXL3Group
from .linear import EXL3Linear
from .moe import glu

_ACTIVATIONS = ("silu", "gelu")


class EXL3MLPMonolith(torch.nn.Module):
    """``down(act(gate(x)) * up(x))`` for EXL3 layers; x (..., in) -> (..., out_of_down) fp16."""

    def __init__(self, group: FusedEXL3Group, down: EXL3Linear, *, activation: str = "silu"):
        super().__init__()
        if activation not in _ACTIVATIONS:
            raise ValueError(f"unsupported MLP activation {activation!r}")
        outs = list(group._out_features)
        if len(outs) != 2 or outs[0] != outs[1]:
            raise ValueError("the gate/up group needs two members of equal width")
        if down.in_features != outs[0]:
            raise ValueError(f"down projection expects {down.in_features} features, gate/up give {outs[0]}")
        self.__dict__["_group"] = group
        self.__dict__["_down"] = down
        self.in_features = group.in_features
        self.hidden_dims = outs[0]
        self.out_features = down.out_features
        self.activation = activation
        self.pdl = False

    @classmethod
    def from_fused_gate_up(cls, group: FusedEXL3Group, down: EXL3Linear, *,
                           activation: str = "silu") -> "EXL3MLPMonolith":
        return cls(group, down, activation=activation)

    def extra_repr(self) -> str:
        return f"in={self.in_features}, hidden={self.hidden_dims}, out={self.out_features}, act={self.activation}"

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[-1] != self.in_features:
            raise ValueError(f"x has {x.shape[-1]} features, the MLP expects {self.in_features}")
        lead = x.shape[:-1]
        x2d = x.reshape(-1, self.in_features)
        rows = x2d.shape[0]
        d = self._down
        if rows == 0:
            return torch.empty(lead + (self.out_features,), dtype=torch.float16, device=x.device)
        if rows <= 16:
            self._group.pdl = self.pdl
            gu = self._group.forward_packed(x2d)                       # (rows, 2 * hidden) = [gate | up]
            y = ops.gemv(gu, d._trellis, d.k, d.cb, d._suh, d._svh, d._bias, pdl=self.pdl,
                         fast_accum=d.fast_accum, glu=self.activation)
        else:
            g, u = self._group.forward_all(x2d)
            if self.activation == "silu":
                h = ops.swiglu(torch.cat([g, u], dim=1))
            else:
                h = glu(g, u, self.activation)
            y = d(h)
        return y.reshape(lead + (self.out_features,))
