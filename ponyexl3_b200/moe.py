"""EXL3 MoE experts — stacked-expert SwitchGLU and the routed block around it.

Mirrors ``EXL3SwitchGLU`` / ``EXL3MoEBlock`` of the reference
(ponyexl3/mlx/exl3_moe.py:425-839).  Per layer the expert trellises are stacked along the
out-tile axis into ONE device buffer — ``gu_trellis (D/16, E*2*H/16, 16K)`` holds all gates,
then all ups; ``dn_trellis (H/16, E*D/16, 16K)`` — with per-expert sign vectors
``gu_suh (E, 2, D)``, ``gu_svh (E, 2H)``, ``dn_suh (E, H)``, ``dn_svh (E, D)``.

``__call__(x (B, S, D), indices (B, S, k)) -> (B, S, k, D)``: un-weighted expert outputs, as
mlx_lm's SwitchGLU; routing and the weighted sum stay in the block.

Decode-class calls (few tokens) run two streamed GEMVs over block tables built on the device
from the routing indices — every (token, slot) pair is its own one-row problem against its
expert's column range (the reference's mapped GEMV, exl3_moe.py:634-683).  Prefill-class
calls sort the pairs by expert and run the tensor-core GEMM over a table of expert tiles
(the reference's segmented trellis GEMM, exl3_moe.py:685-768).
"""

from __future__ import annotations

import torch

from . import ops

_ACTIVATIONS = ("silu", "gelu")
DECODE_MAX_TOKENS = 16


def glu(g: torch.Tensor, u: torch.Tensor, activation: str) -> torch.Tensor:
    """fp16( act(g) * u ), float32 math (ponyexl3/mlx/exl3_moe.py:62-75)."""
    g32, u32 = g.float(), u.float()
    if activation == "gelu":
        h = 0.5 * g32 * (1.0 + torch.tanh(0.797884560803 * (g32 + 0.044715 * g32 * g32 * g32))) * u32
    else:
        h = (g32 / (1.0 + torch.exp(-g32))) * u32
    return h.to(torch.float16)


class EXL3SwitchGLU(torch.nn.Module):
    """Stacked-expert EXL3 SwitchGLU (gate+up per expert, then down)."""

    def __init__(self, *, gu_trellis: torch.Tensor, gu_suh: torch.Tensor, gu_svh: torch.Tensor,
                 dn_trellis: torch.Tensor, dn_suh: torch.Tensor, dn_svh: torch.Tensor, k: int, cb: int,
                 activation: str = "silu"):
        super().__init__()
        if activation not in _ACTIVATIONS:
            raise ValueError(f"unsupported MoE activation {activation!r}")
        if not gu_trellis.is_cuda:
            raise RuntimeError("EXL3SwitchGLU needs CUDA tensors: there is no CPU path")
        self.num_experts = int(gu_suh.shape[0])
        self.input_dims = int(gu_suh.shape[2])
        self.hidden_dims = int(dn_suh.shape[1])
        E, D, H = self.num_experts, self.input_dims, self.hidden_dims
        if D % 128 or H % 128:
            raise ValueError("expert dims must be multiples of 128")
        if tuple(gu_trellis.shape) != (D // 16, E * 2 * H // 16, 16 * k):
            raise ValueError(f"gu_trellis shape {tuple(gu_trellis.shape)} does not fit E={E} D={D} H={H} K={k}")
        if tuple(dn_trellis.shape) != (H // 16, E * D // 16, 16 * k):
            raise ValueError(f"dn_trellis shape {tuple(dn_trellis.shape)} does not fit E={E} D={D} H={H} K={k}")
        if tuple(gu_svh.shape) != (E, 2 * H) or tuple(dn_svh.shape) != (E, D) or tuple(dn_suh.shape) != (E, H):
            raise ValueError("sign vector shapes do not fit the expert dims")
        self.k, self.cb, self.activation = int(k), int(cb), activation
        self._gu_trellis = gu_trellis.contiguous()
        self._dn_trellis = dn_trellis.contiguous()
        self._gu_suh = gu_suh.to(torch.float16).reshape(E * 2, D).contiguous()
        self._gu_svh = gu_svh.to(torch.float16).reshape(-1).contiguous()
        self._dn_suh = dn_suh.to(torch.float16).contiguous()
        self._dn_svh = dn_svh.to(torch.float16).reshape(-1).contiguous()
        self.pdl = False

    # ---- decode: every (token, slot) pair is a one-row problem -------------------------------
    def _decode(self, x2d: torch.Tensor, indices: torch.Tensor, expert_range=None) -> torch.Tensor:
        """Three launches: tables, GEMV over (pair, gate|up) blocks, GEMV over (pair, down) blocks
        with the GLU folded into its activation load (the reference's two-launch fused decode,
        ponyexl3/mlx/exl3_moe.py:345-422).  No host round trip, so the call can be captured.

        expert_range = (lo, hi, total): this module holds experts lo..hi-1 of `total`, `indices`
        are global; only the pairs of held experts are computed (their number stays on the device),
        the rows of all other pairs come back as zeros."""
        from . import _lib
        E, D, H = self.num_experts, self.input_dims, self.hidden_dims
        R, kk = indices.shape
        n = R * kk
        dev = x2d.device
        gb, db = H // 128, D // 128
        idx = indices.reshape(-1)
        if idx.dtype not in (torch.int32, torch.int64):
            idx = idx.to(torch.int64)
        idx = idx.contiguous()
        # one int32 buffer: blocks_gu | blocks_dn | row_src_gu | suh_row_gu | suh_row_dn | counts
        n_gu, n_dn = n * 2 * gb * 4, n * db * 4
        tab = torch.empty(n_gu + n_dn + 5 * n + 4, dtype=torch.int32, device=dev)
        blocks_gu, blocks_dn = tab[:n_gu].view(-1, 4), tab[n_gu:n_gu + n_dn].view(-1, 4)
        o = n_gu + n_dn
        row_src, suh_row, sel = tab[o:o + 2 * n], tab[o + 2 * n:o + 4 * n], tab[o + 4 * n:o + 5 * n]
        counts = tab[o + 5 * n:o + 5 * n + 2]
        flags = _lib.FLAG_PDL if self.pdl else 0
        stream = torch.cuda.current_stream(dev).cuda_stream
        if expert_range is None:
            _lib.check(_lib.load().exl3_moe_decode_tables(
                idx.data_ptr(), idx.element_size(), n, kk, E, D, H, blocks_gu.data_ptr(), row_src.data_ptr(),
                suh_row.data_ptr(), blocks_dn.data_ptr(), sel.data_ptr(), flags, stream), "exl3_moe_decode_tables")
            cnt_gu = cnt_dn = None
            new = torch.empty
        else:
            lo, hi, total = expert_range
            if hi - lo != E:
                raise ValueError("expert_range does not match the experts held here")
            _lib.check(_lib.load().exl3_moe_decode_tables_range(
                idx.data_ptr(), idx.element_size(), n, kk, total, lo, hi, D, H, blocks_gu.data_ptr(),
                row_src.data_ptr(), suh_row.data_ptr(), blocks_dn.data_ptr(), sel.data_ptr(), counts.data_ptr(),
                flags, stream), "exl3_moe_decode_tables_range")
            cnt_gu, cnt_dn = counts[0:1], counts[1:2]
            new = torch.zeros

        ygu = torch.empty((n, 2 * H), dtype=torch.float16, device=dev)   # rows of other ranks' pairs: never read
        ops.gemv_blocks(x2d, xh_rows=2 * n, row_src=row_src, suh=self._gu_suh, suh_row=suh_row,
                        trellis=self._gu_trellis, k=self.k, cb=self.cb, blocks=blocks_gu, rows=1,
                        svh=self._gu_svh, bias=None, y=ygu, pdl=self.pdl, n_blocks_dev=cnt_gu)
        # the down launch reads [gate | up] as it is and applies the GLU while loading
        y = new((n, D), dtype=torch.float16, device=dev)
        ops.gemv_blocks(ygu, xh_rows=n, row_src=None, suh=self._dn_suh, suh_row=sel,
                        trellis=self._dn_trellis, k=self.k, cb=self.cb, blocks=blocks_dn, rows=1,
                        svh=self._dn_svh, bias=None, y=y, pdl=self.pdl, glu=self.activation,
                        n_blocks_dev=cnt_dn)
        return y.view(R, kk, D)

    @torch.no_grad()
    def decode_range(self, x2d: torch.Tensor, indices: torch.Tensor, expert_range) -> torch.Tensor:
        """Expert parallelism, few tokens: this module holds experts lo..hi-1 of `total`
        (expert_range = (lo, hi, total)), `indices` (R, k) are global.  Returns (R, k, D) with the
        rows of pairs routed elsewhere zero, so the ranks' results add up to the full output."""
        if indices.shape[0] > DECODE_MAX_TOKENS:
            raise ValueError("decode_range is for decode-class calls")
        return self._decode(x2d, indices, expert_range)

    # ---- prefill: pairs sorted by expert, tensor-core GEMM over an expert tile table ----------
    def _prefill(self, x2d: torch.Tensor, indices: torch.Tensor, expert_range=None, peers=None):
        """Tables kernel, rotation + tile-table GEMM for gate and up, rotation (GLU applied while
        loading) + tile-table GEMM for down writing straight back into (token, slot) order: five
        launches, no host round trip.

        expert_range = (lo, hi, total) and peers = (y_ptrs, counter_ptrs, n, rows_per_peer,
        row_stride): expert parallelism — this module holds experts lo..hi-1, `indices` are global
        and cover ALL tokens; only the held pairs are computed (their number stays on the device)
        and every output row is stored into the memory of the GPU that owns its token, which
        gets one arrival per GPU when the rows are complete (exl3_gemm_tiles_peers)."""
        from . import _lib
        E, D, H = self.num_experts, self.input_dims, self.hidden_dims
        R, kk = indices.shape
        n = R * kk
        dev = x2d.device
        idx = indices.reshape(-1)
        if idx.dtype not in (torch.int32, torch.int64):
            idx = idx.to(torch.int64)
        idx = idx.contiguous()
        slots = n // 256 + E
        ct_h, ct_d = (H + 255) // 256, (D + 255) // 256
        n_gu, n_dn = 2 * slots * ct_h * 8, slots * ct_d * 8
        tab = torch.empty(n_gu + n_dn + 6 * n + 4, dtype=torch.int32, device=dev)   # tiles first: 16-byte aligned
        tiles_gu, tiles_dn = tab[:n_gu].view(-1, 8), tab[n_gu:n_gu + n_dn].view(-1, 8)
        o = n_gu + n_dn
        order, row_src = tab[o:o + n], tab[o + n:o + 3 * n]
        suh_gu, suh_dn = tab[o + 3 * n:o + 5 * n], tab[o + 5 * n:o + 6 * n]
        counts = tab[o + 6 * n:o + 6 * n + 2]
        stream = torch.cuda.current_stream(dev).cuda_stream
        if expert_range is None:
            _lib.check(_lib.load().exl3_moe_prefill_tables(
                idx.data_ptr(), idx.element_size(), n, kk, E, D, H, order.data_ptr(), row_src.data_ptr(),
                suh_gu.data_ptr(), suh_dn.data_ptr(), tiles_gu.data_ptr(), tiles_dn.data_ptr(), 0, stream),
                "exl3_moe_prefill_tables")
            rows_gu = rows_dn = None
        else:
            lo, hi, total = expert_range
            if hi - lo != E:
                raise ValueError("expert_range does not match the experts held here")
            _lib.check(_lib.load().exl3_moe_prefill_tables_range(
                idx.data_ptr(), idx.element_size(), n, kk, total, lo, hi, D, H, order.data_ptr(), row_src.data_ptr(),
                suh_gu.data_ptr(), suh_dn.data_ptr(), tiles_gu.data_ptr(), tiles_dn.data_ptr(), counts.data_ptr(),
                0, stream), "exl3_moe_prefill_tables_range")
            rows_gu, rows_dn = counts[0:1], counts[1:2]
        ygu = torch.empty((n, 2 * H), dtype=torch.float16, device=dev)
        ops.gemm_tiles(x2d, xh_rows=2 * n, row_src=row_src, suh=self._gu_suh, suh_row=suh_gu,
                       trellis=self._gu_trellis, k=self.k, cb=self.cb, tiles=tiles_gu, svh=self._gu_svh, y=ygu,
                       xh_rows_dev=rows_gu)
        # the down launch reads [gate | up] as it is and applies the GLU while it rotates the rows
        out = None if peers is not None else torch.empty((n, D), dtype=torch.float16, device=dev)
        ops.gemm_tiles(ygu, xh_rows=n, row_src=None, suh=self._dn_suh, suh_row=suh_dn, trellis=self._dn_trellis,
                       k=self.k, cb=self.cb, tiles=tiles_dn, svh=self._dn_svh, y=out, y_row_map=order,
                       glu=self.activation, xh_rows_dev=rows_dn, peers=peers)
        return None if out is None else out.view(R, kk, D)

    @torch.no_grad()
    def prefill_range(self, x2d: torch.Tensor, indices: torch.Tensor, expert_range, peers) -> None:
        """Expert parallelism, many tokens: see _prefill.  x2d (T, D) and indices (T, k) cover all
        tokens; the outputs land in the owners' buffers named by `peers`."""
        self._prefill(x2d, indices, expert_range, peers)

    @torch.no_grad()
    def forward(self, x: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
        if indices.ndim != 3:
            raise ValueError("indices must be (B, S, k)")
        B, S, kk = indices.shape
        R = B * S
        x2d = x.reshape(R, self.input_dims)
        idx = indices.reshape(R, kk)
        y = self._decode(x2d, idx) if R <= DECODE_MAX_TOKENS else self._prefill(x2d, idx)
        return y.reshape(B, S, kk, self.input_dims)


def route_topk(logits: torch.Tensor, top_k: int, norm_topk_prob: bool = True):
    """softmax -> top-k -> renormalise (ponyexl3/mlx/exl3_moe.py:807-831): indices, scores."""
    gates = torch.softmax(logits.float(), dim=-1)
    scores, inds = torch.topk(gates, top_k, dim=-1)
    if norm_topk_prob:
        scores = scores / scores.sum(dim=-1, keepdim=True)
    return inds, scores


class EXL3MoEBlock(torch.nn.Module):
    """Router + stacked experts + weighted sum (ponyexl3/mlx/exl3_moe.py:790-839).

    With `shared_gate_weight` the shared expert is stacked as the LAST expert of the switch and
    its gate value sigmoid(x @ shared_gate_weight.T) is one more routing weight: every token gets
    the slot (num_experts - 1) appended to its top-k (the reference's Qwen3-Next block, :790-798,
    :823-829)."""

    def __init__(self, gate_weight: torch.Tensor, switch, top_k: int, norm_topk_prob: bool = True,
                 shared_gate_weight: torch.Tensor | None = None):
        super().__init__()
        self.gate_weight = gate_weight          # (E or E - 1, D) router, unquantised
        self.shared_gate_weight = shared_gate_weight    # (1, D) or None
        self.switch_mlp = switch
        self.top_k = top_k
        self.norm_topk_prob = norm_topk_prob

    def route(self, x3: torch.Tensor):
        """(indices (1, T, k or k + 1), scores): the routing decision alone."""
        inds, scores = route_topk(x3.float() @ self.gate_weight.float().t(), self.top_k, self.norm_topk_prob)
        if self.shared_gate_weight is not None:
            shared_idx = self.switch_mlp.num_experts - 1
            shared_w = torch.sigmoid(x3.float() @ self.shared_gate_weight.float().t())
            inds = torch.cat([inds, torch.full_like(inds[..., :1], shared_idx)], dim=-1)
            scores = torch.cat([scores.to(x3.dtype).float(), shared_w], dim=-1)
        return inds, scores

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x3 = x.reshape(1, -1, x.shape[-1])
        inds, scores = self.route(x3)
        y = self.switch_mlp(x3, inds)
        return (y.float() * scores[..., None]).sum(dim=-2).to(torch.float16).reshape(lead + (x.shape[-1],))


class EXL3Gemma4MoEBlock(torch.nn.Module):
    """Gemma4's router in front of the stacked experts (ponyexl3/mlx/exl3_moe.py:842-923): RMS norm
    of the hidden state with weight scale * hidden_size**-0.5, a linear projection to expert
    scores, top-k of the RAW scores, softmax over the selected k, times a per-expert scale.
    Called with x alone it returns (indices, weights) as the reference's router slot does; called
    with the routing it runs the experts and the weighted sum."""

    def __init__(self, proj_weight: torch.Tensor, scale: torch.Tensor, per_expert_scale: torch.Tensor, switch,
                 top_k: int, eps: float, hidden_size: int):
        super().__init__()
        self.proj_weight = proj_weight          # (E, D)
        self.scale = scale                      # (D,)
        self.per_expert_scale = per_expert_scale  # (E,)
        self.switch_mlp = switch
        self.top_k = top_k
        self.eps = eps
        self._root_scale = hidden_size ** -0.5

    def route(self, h: torch.Tensor):
        h32 = h.float()
        normed = h32 * torch.rsqrt(h32.pow(2).mean(dim=-1, keepdim=True) + self.eps) * (self.scale.float() * self._root_scale)
        expert_scores = normed @ self.proj_weight.float().t()
        weights, inds = torch.topk(expert_scores, self.top_k, dim=-1)
        weights = torch.softmax(weights, dim=-1) * self.per_expert_scale.float()[inds]
        return inds, weights

    @torch.no_grad()
    def forward(self, x: torch.Tensor, top_k_indices: torch.Tensor | None = None,
                top_k_weights: torch.Tensor | None = None):
        if top_k_indices is None:
            return self.route(x)
        lead = x.shape[:-1]
        x3 = x.reshape(1, -1, x.shape[-1])
        kk = top_k_indices.shape[-1]
        y = self.switch_mlp(x3, top_k_indices.reshape(1, -1, kk))
        w = top_k_weights.reshape(1, -1, kk).float()
        return (w[..., None] * y.float()).sum(dim=-2).to(torch.float16).reshape(lead + (x.shape[-1],))
