"""The synthetic decode step with its glue (RMSNorm, rotary embedding, attention over the KV
cache, SiLU-GLU) written as plain PyTorch ops — the comparator for the library's step kernels.
The EXL3 linears still run through the library; only what sits between them differs."""

from __future__ import annotations

import torch
import torch.nn.functional as F

from ponyexl3_b200.dense_step import SyntheticDenseDecoder


class TorchGlueDecoder(SyntheticDenseDecoder):
    def __init__(self, *args, **kwargs):
        kwargs["peer_exchange"] = False
        super().__init__(*args, **kwargs)
        self._masks: dict[int, torch.Tensor] = {}

    def _rope(self, t: torch.Tensor, rows: int) -> torch.Tensor:
        """t (rows, heads, hd): rotate-half RoPE at positions context .. context+rows-1."""
        cos, sin = self.cos[:rows, None, :], self.sin[:rows, None, :]
        half = t.shape[-1] // 2
        rot = torch.cat([-t[..., half:], t[..., :half]], dim=-1)
        return t * cos + rot * sin

    def _mask(self, rows: int) -> torch.Tensor | None:
        """Row (g, r) of the folded query block sees cache positions <= context + r."""
        if rows == 1:
            return None
        m = self._masks.get(rows)
        if m is None:
            c = self.cfg
            kpos = torch.arange(c.context + rows, device=self.dev)
            qpos = c.context + torch.arange(rows, device=self.dev)
            m = (kpos[None, :] <= qpos[:, None]).repeat(c.group, 1)        # (group*rows, L)
            self._masks[rows] = m
        return m

    def _attention(self, L, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rows: int):
        """q (rows, hq, hd), k/v (rows, hkv, hd) of the new positions -> (rows, hq*hd)."""
        c = self.cfg
        end = c.context + rows
        L.k_cache[:, c.context:end] = k.transpose(0, 1)
        L.v_cache[:, c.context:end] = v.transpose(0, 1)
        # fold the query heads of one KV head into the query length: (1, hkv, group*rows, hd)
        qf = q.view(rows, self.hkv, c.group, c.head_dim).permute(1, 2, 0, 3).reshape(
            1, self.hkv, c.group * rows, c.head_dim)
        out = F.scaled_dot_product_attention(qf, L.k_cache[None, :, :end], L.v_cache[None, :, :end],
                                             attn_mask=self._mask(rows))
        return out.view(self.hkv, c.group, rows, c.head_dim).permute(2, 0, 1, 3).reshape(rows, -1)

    @torch.no_grad()
    def forward_logits(self, tokens: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        rows = tokens.shape[0]
        hd = c.head_dim
        x = self.embed[tokens]                                            # (rows, hidden)
        for L in self.layers:
            h = F.rms_norm(x, (c.hidden,), L.norm1, c.rms_eps)
            q, k, v = L.qkv.forward_all(h)
            q = self._rope(q.reshape(rows, self.hq, hd), rows)
            k = self._rope(k.reshape(rows, self.hkv, hd), rows)
            a = self._attention(L, q, k, v.reshape(rows, self.hkv, hd), rows)
            a = self._gather(a, [(r * self.hq * hd, (r + 1) * self.hq * hd) for r in range(self.world)])
            x = x + self._gather(L.o(a), self.hidden_spans)
            h = F.rms_norm(x, (c.hidden,), L.norm2, c.rms_eps)
            g, u = L.gate_up.forward_all(h)
            act = self._gather(F.silu(g) * u, self.inter_spans)
            x = x + self._gather(L.down(act), self.hidden_spans)
        h = F.rms_norm(x, (c.hidden,), self.final_norm, c.rms_eps)
        return self.head(h)
