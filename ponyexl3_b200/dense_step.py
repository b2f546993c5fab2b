"""One greedy decode step of a synthetic dense transformer whose linears are all EXL3.

This is the caller that sits on both sides of the EXL3 path during generation: the model graph
the reference hands to mlx_lm (ponyexl3/mlx/model.py:628-634 installs an EXL3Linear on every
linear slot; ponyexl3/mlx/exl3_fused.py:92-211 groups q/k/v and gate/up).  Here it exists to
measure the path in its real setting — 64 layers of q/k/v, o, gate/up, down plus the vocabulary
head, grouped-query attention over a long KV context between them — with random weights of the
right shapes.  Every linear runs through the library's GEMV entry points; residual + RMSNorm,
RoPE + cache append, grouped-query attention and the GLU are the library's step kernels
(exl3_step.cu), so a step is a short train of launches; only the embedding gather and the final
arg-max are PyTorch ops.

Tensor parallel layout (one process per GPU): every linear is sharded by OUTPUT TILE.
q/k/v are cut by head, so attention needs no collective; the attention output, the o_proj
output, the SwiGLU output and the down output are each all-gathered (4 per layer).  The head
is cut into 128-column blocks (1187 of them, uneven) and reduced by an arg-max exchange.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist

from .fused import FusedEXL3Group
from .linear import EXL3Linear
from .parallel import shard_blocks


@dataclass
class DenseConfig:
    layers: int = 64
    hidden: int = 5120
    intermediate: int = 17408
    q_heads: int = 40
    kv_heads: int = 8
    head_dim: int = 128
    vocab: int = 151936
    context: int = 8192            # KV positions already in the cache
    max_rows: int = 16             # new positions per step (1 = decode, 16 = speculative verify)
    rms_eps: float = 1e-6
    rope_theta: float = 1_000_000.0
    k5_fraction: float = 0.15      # share of linears at K=5, the rest K=4 (mean ~4.15 bpw)
    codebook: int = 0

    @property
    def group(self) -> int:
        return self.q_heads // self.kv_heads

    def packed_bytes(self, ks: list[int]) -> int:
        """Packed weight bytes of the whole model for per-slot K values `ks` (4 slots per layer
        in the order qkv, o, gate/up, down, then the head)."""
        d, i, hd = self.hidden, self.intermediate, self.head_dim
        per_slot = [d * (self.q_heads + 2 * self.kv_heads) * hd, self.q_heads * hd * d, d * 2 * i, i * d]
        total = 0
        for layer in range(self.layers):
            for s in range(4):
                total += per_slot[s] * ks[4 * layer + s] // 8
        return total + d * self.vocab * ks[-1] // 8


def draw_bit_widths(cfg: DenseConfig, seed: int) -> list[int]:
    """K per linear slot, seeded; sibling linears that are launched as one group share a K."""
    g = torch.Generator()
    g.manual_seed(seed)
    u = torch.rand(4 * cfg.layers + 1, generator=g)
    return [5 if v < cfg.k5_fraction else 4 for v in u.tolist()]


def _rand_trellis(t_in: int, t_out: int, k: int, dev, gen) -> torch.Tensor:
    return torch.randint(-32768, 32767, (t_in, t_out, 16 * k), dtype=torch.int16, device=dev, generator=gen)


def _rand_signs(n, dev, gen) -> torch.Tensor:
    shape = n if isinstance(n, tuple) else (n,)
    return (torch.randint(0, 2, shape, device=dev, generator=gen) * 2 - 1).to(torch.float16)


class _Layer:
    __slots__ = ("qkv", "o", "gate_up", "down", "mlp", "norm1", "norm2", "k_cache", "v_cache")


class SyntheticDenseDecoder:
    """Random-weight dense decoder with a pre-filled KV cache; `step(tokens)` runs one forward
    over `rows` new positions and returns the arg-max token of every row."""

    def __init__(self, cfg: DenseConfig, device: torch.device, seed: int = 5000, group=None,
                 pdl: bool = True, tensor_parallel: bool = True, peer_exchange: bool = True):
        self.cfg, self.dev, self.pg = cfg, device, group
        if cfg.head_dim != 128:
            raise ValueError("the step kernels (rotary, attention) serve head_dim 128 only")
        self.pdl_glue = pdl
        self.world = (dist.get_world_size(group)
                      if (tensor_parallel and dist.is_available() and dist.is_initialized()) else 1)
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        W, R = self.world, self.rank
        # peer_exchange: the four all-gathers of a layer go over peer memory (the o / down GEMVs
        # store their blocks into every rank's row, attention and SwiGLU outputs are copied the same
        # way); otherwise NCCL all-gathers
        self.peer = None
        if W > 1 and peer_exchange:
            from .parallel import PeerExchange
            self.peer = PeerExchange(cfg.max_rows, max(cfg.intermediate, cfg.q_heads * cfg.head_dim),
                                     group, ring=PeerExchange.ring_for(4 * cfg.layers))
        if cfg.kv_heads % W:
            raise ValueError(f"{cfg.kv_heads} KV heads do not split over {W} ranks")
        self.ks = draw_bit_widths(cfg, seed)
        # Every rank draws the WHOLE tensor from the same seeded generator and keeps its column
        # slice, so the sharded model is the same model at every world size.
        gen = torch.Generator(device=device)
        gen.manual_seed(seed)
        d, hd = cfg.hidden, cfg.head_dim
        self.hq, self.hkv = cfg.q_heads // W, cfg.kv_heads // W
        qn, kvn = self.hq * hd, self.hkv * hd
        blocks = lambda n, r: tuple(128 * v for v in shard_blocks(n // 128, W, r))
        self.inter_spans = [blocks(cfg.intermediate, r) for r in range(W)]
        self.hidden_spans = [blocks(d, r) for r in range(W)]
        i0, i1 = self.inter_spans[R]
        d0, d1 = self.hidden_spans[R]
        self.inter_local = i1 - i0
        cb = cfg.codebook
        scale = lambda n_in: 1.0 / (1.25 * math.sqrt(n_in))       # keeps activations near unit scale

        def columns(n_in, n_out, k, spans):
            """(trellis, svh) of a full (n_in -> n_out) linear, cut to the column spans given."""
            tr = _rand_trellis(n_in // 16, n_out // 16, k, device, gen)
            sv = _rand_signs(n_out, device, gen) * scale(n_in)
            if W == 1:
                return tr, sv
            return (torch.cat([tr[:, a // 16:b // 16] for a, b in spans], dim=1).contiguous(),
                    torch.cat([sv[a:b] for a, b in spans]))

        self.layers: list[_Layer] = []
        self.packed_local = 0
        length = cfg.context + cfg.max_rows
        q_all, kv_all = cfg.q_heads * hd, cfg.kv_heads * hd
        for li in range(cfg.layers):
            L = _Layer()
            k_qkv, k_o, k_gu, k_dn = self.ks[4 * li:4 * li + 4]
            # q | k | v side by side; this rank keeps its heads of each
            tr, sv = columns(d, q_all + 2 * kv_all, k_qkv,
                             [(R * qn, (R + 1) * qn), (q_all + R * kvn, q_all + (R + 1) * kvn),
                              (q_all + kv_all + R * kvn, q_all + kv_all + (R + 1) * kvn)])
            L.qkv = FusedEXL3Group.from_device_tensors(
                trellis=tr, k=k_qkv, cb=cb, suh_stack=_rand_signs((3, d), device, gen), svh_cat=sv,
                out_features=[qn, kvn, kvn], keys=[f"l{li}.q", f"l{li}.k", f"l{li}.v"])
            tr, sv = columns(q_all, d, k_o, [(d0, d1)])
            L.o = EXL3Linear.from_device_tensors(trellis=tr, k=k_o, cb=cb, suh=_rand_signs(q_all, device, gen),
                                                 svh=sv, key=f"l{li}.o")
            tr, sv = columns(d, 2 * cfg.intermediate, k_gu,
                             [(i0, i1), (cfg.intermediate + i0, cfg.intermediate + i1)])
            L.gate_up = FusedEXL3Group.from_device_tensors(
                trellis=tr, k=k_gu, cb=cb, suh_stack=_rand_signs((2, d), device, gen), svh_cat=sv,
                out_features=[self.inter_local, self.inter_local], keys=[f"l{li}.gate", f"l{li}.up"])
            tr, sv = columns(cfg.intermediate, d, k_dn, [(d0, d1)])
            L.down = EXL3Linear.from_device_tensors(trellis=tr, k=k_dn, cb=cb,
                                                    suh=_rand_signs(cfg.intermediate, device, gen), svh=sv,
                                                    key=f"l{li}.down")
            # one GPU: gate|up -> GLU -> down as two launches (the GLU rides the down kernel's load)
            L.mlp = None
            if W == 1:
                from .mlp import EXL3MLPMonolith
                L.mlp = EXL3MLPMonolith(L.gate_up, L.down)
            for m in (L.qkv, L.o, L.gate_up, L.down):
                m.pdl = pdl and (W == 1 or self.peer is not None)   # between NCCL kernels: plain stream order
                self.packed_local += m.packed_bytes
            L.norm1 = torch.ones(d, dtype=torch.float16, device=device)
            L.norm2 = torch.ones(d, dtype=torch.float16, device=device)
            kc = torch.randn((cfg.kv_heads, length, hd), device=device, generator=gen).to(torch.float16)
            vc = torch.randn((cfg.kv_heads, length, hd), device=device, generator=gen).to(torch.float16)
            L.k_cache = kc[R * self.hkv:(R + 1) * self.hkv].contiguous()
            L.v_cache = vc[R * self.hkv:(R + 1) * self.hkv].contiguous()
            self.layers.append(L)
        # vocabulary head, cut into 128-column blocks (uneven split)
        self.vocab_span = blocks(cfg.vocab, R)
        k_head = self.ks[-1]
        tr, sv = columns(d, cfg.vocab, k_head, [self.vocab_span])
        self.head = EXL3Linear.from_device_tensors(trellis=tr, k=k_head, cb=cb, suh=_rand_signs(d, device, gen),
                                                   svh=sv, key="lm_head")
        self.head.pdl = pdl and (W == 1 or self.peer is not None)
        self.packed_local += self.head.packed_bytes
        self.final_norm = torch.ones(d, dtype=torch.float16, device=device)
        self.embed = torch.randn((cfg.vocab, d), device=device, generator=gen).to(torch.float16)
        # rotary tables for the new positions context .. context+max_rows-1
        pos = torch.arange(cfg.context, cfg.context + cfg.max_rows, device=device, dtype=torch.float32)
        inv = cfg.rope_theta ** (-torch.arange(0, hd, 2, device=device, dtype=torch.float32) / hd)
        ang = pos[:, None] * inv[None, :]
        self.cos = torch.cat([ang.cos(), ang.cos()], dim=-1).to(torch.float16)     # (max_rows, hd)
        self.sin = torch.cat([ang.sin(), ang.sin()], dim=-1).to(torch.float16)

    # ---- pieces ------------------------------------------------------------------------------
    @property
    def kv_bytes_local(self) -> int:
        c = self.cfg
        return c.layers * 2 * self.hkv * c.context * c.head_dim * 2

    def _gather(self, y_local: torch.Tensor, spans) -> torch.Tensor:
        """All-gather of column shards (rows, local) -> (rows, total); identity on one rank."""
        if self.world == 1:
            return y_local
        rows = y_local.shape[0]
        widths = [b - a for a, b in spans]
        if len(set(widths)) == 1:
            full = torch.empty((self.world, rows, widths[0]), dtype=y_local.dtype, device=y_local.device)
            dist.all_gather_into_tensor(full.view(-1), y_local.contiguous().view(-1), group=self.pg)
            return full.view(rows, -1) if rows == 1 else full.permute(1, 0, 2).reshape(rows, -1)
        wmax = max(widths)
        pad = torch.zeros((rows, wmax), dtype=y_local.dtype, device=y_local.device)
        pad[:, :y_local.shape[1]] = y_local
        full = torch.empty((self.world, rows, wmax), dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(full.view(-1), pad.view(-1), group=self.pg)
        return torch.cat([full[r, :, :w] for r, w in enumerate(widths)], dim=1)

    # ---- the step ----------------------------------------------------------------------------
    def _forward_native(self, tokens: torch.Tensor) -> torch.Tensor:
        """The step with the library's glue kernels: 13 launches per layer on one GPU."""
        from . import ops
        c = self.cfg
        rows = tokens.shape[0]
        q_all = c.q_heads * 128
        peer = self.peer
        if peer is not None:
            peer.restart()
        pdl = self.pdl_glue

        def gather(t, spans, total):
            # the gathered row is read by the GEMV that follows: its kernel waits for the arrivals
            # itself, no wait launch in between
            if peer is None:
                return self._gather(t, spans)
            return ops.peer_allgather(t, exchange=peer, cols_total=total, col0=spans[self.rank][0], pdl=pdl,
                                      defer_wait=True)

        def linear_gather(m, t, spans, total):
            if peer is None:
                return self._gather(m(t), spans)
            return ops.gemv_peers(t, m._trellis, m.k, m.cb, m._suh, m._svh, m._bias, exchange=peer,
                                  out_features_total=total, col0=spans[self.rank][0], pdl=m.pdl)

        head_spans = [(r * self.hq * 128, (r + 1) * self.hq * 128) for r in range(self.world)]
        x = self.embed[tokens]                                            # (rows, hidden), updated in place
        delta = None
        for L in self.layers:
            h = ops.add_rmsnorm(x, delta, L.norm1, c.rms_eps, pdl=pdl)
            qkv = L.qkv.forward_packed(h)
            q = ops.rope_append(qkv, self.cos, self.sin, L.k_cache, L.v_cache, self.hq, c.context, pdl=pdl)
            a = gather(ops.attn_decode(q, L.k_cache, L.v_cache, c.context, pdl=pdl), head_spans, q_all)
            o = linear_gather(L.o, a, self.hidden_spans, c.hidden)
            h = ops.add_rmsnorm(x, o, L.norm2, c.rms_eps, pdl=pdl)
            if L.mlp is not None and rows <= 16:
                L.mlp.pdl = L.down.pdl
                delta = L.mlp(h)
            else:
                act = gather(ops.swiglu(L.gate_up.forward_packed(h), pdl=pdl), self.inter_spans, c.intermediate)
                delta = linear_gather(L.down, act, self.hidden_spans, c.hidden)
        h = ops.add_rmsnorm(x, delta, self.final_norm, c.rms_eps, pdl=pdl)
        return self.head(h)

    @torch.no_grad()
    def forward_logits(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens (rows,) int64 -> this rank's slice of the logits (rows, local vocab) fp16."""
        return self._forward_native(tokens)

    @torch.no_grad()
    def step(self, tokens: torch.Tensor) -> torch.Tensor:
        """One greedy step: the arg-max token of every row, identical on every rank."""
        rows = tokens.shape[0]
        logits = self.forward_logits(tokens)
        best, arg = logits.float().max(dim=-1)
        arg = arg + self.vocab_span[0]
        if self.world == 1:
            return arg
        pair = torch.stack([best, arg.float()], dim=-1).contiguous()      # token ids < 2**24: exact
        allp = torch.empty((self.world,) + pair.shape, dtype=pair.dtype, device=pair.device)
        dist.all_gather_into_tensor(allp.view(-1), pair.view(-1), group=self.pg)
        win = allp[..., 0].argmax(dim=0)                                  # (rows,)
        return allp[win, torch.arange(rows, device=self.dev), 1].long()
