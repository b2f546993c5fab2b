"""Sharding of the EXL3 path over the GPUs of one box (one process per GPU, torch.distributed).

The reference is single-device; what has to hold here is only that the sharded result
equals the unsharded one.

* Dense linear — tensor parallel by OUTPUT TILE.  Tiles are independent and stored
  ``[in_tile][out_tile]``, so a rank's shard is a column slice of the packed trellis with no
  re-encoding.  Shards are whole 128-column blocks, which keeps the output Hadamard rotation,
  ``svh`` and ``bias`` local; every rank needs the whole input row and the whole ``suh``.  The
  per-rank outputs are all-gathered (NCCL on GPUs, gloo in the CPU tests).
* Stacked MoE experts — expert parallel: rank g owns a contiguous range of experts (a
  contiguous out-tile range of the stacked trellises).  Decode-class calls replicate the few
  tokens, every rank computes the (token, slot) pairs whose expert it owns — picked and counted
  on the device — and the partial outputs are summed (all-reduce).  Prefill-class calls with
  tokens partitioned over the ranks gather tokens and routing, every rank computes the pairs of
  its experts and stores each output row into the memory of the rank that owns the token
  (``EPSwitchGLU.forward_partitioned``); the same exchange written as two all-to-alls
  (``dispatch_rows_to_experts`` / ``return_rows_to_tokens``) is what the CPU tests run.
"""

from __future__ import annotations

from typing import Callable

import numpy as np
import torch
import torch.distributed as dist

from .layer import EXL3Layer, unpack_signs_or_pass


def shard_blocks(n_blocks: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous block range [b0, b1) of `rank`; the first n_blocks % world ranks get one more."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n_blocks, world)
    b0 = rank * base + min(rank, extra)
    return b0, b0 + base + (1 if rank < extra else 0)


def shard_columns(out_features: int, world: int, rank: int) -> tuple[int, int]:
    """Column range of `rank` under tensor parallelism by output tile (multiples of 128)."""
    if out_features % 128:
        raise ValueError("out_features must be a multiple of 128")
    b0, b1 = shard_blocks(out_features // 128, world, rank)
    return b0 * 128, b1 * 128


def shard_layer(layer: EXL3Layer, world: int, rank: int) -> EXL3Layer:
    """The column shard of `layer` owned by `rank` (may be empty when world > blocks)."""
    c0, c1 = shard_columns(layer.out_features, world, rank)
    svh = unpack_signs_or_pass(layer.svh)
    return EXL3Layer(
        key=f"{layer.key}[tp{rank}/{world}]", in_features=layer.in_features, out_features=c1 - c0,
        k=layer.k, trellis=np.ascontiguousarray(layer.trellis[:, c0 // 16:c1 // 16]), suh=layer.suh,
        svh=None if svh is None else svh[c0:c1],
        bias=None if layer.bias is None else layer.bias[c0:c1], mcg=layer.mcg, mul1=layer.mul1)


def all_gather_columns(y_local: torch.Tensor, out_features: int, group=None) -> torch.Tensor:
    """(rows, local_cols) on every rank -> (rows, out_features) on every rank, for the uneven
    128-block split of shard_columns."""
    world = dist.get_world_size(group)
    rows = y_local.shape[0]
    if (out_features // 128) % world == 0:
        full = torch.empty((world, rows, out_features // world), dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(full.view(-1), y_local.contiguous().view(-1), group=group)
        return full.permute(1, 0, 2).reshape(rows, out_features)
    # uneven split (e.g. 1187 blocks over 8 ranks): pad every shard to the widest, gather, cut
    spans = [shard_columns(out_features, world, r) for r in range(world)]
    wmax = max(c1 - c0 for c0, c1 in spans)
    padded = torch.zeros((rows, wmax), dtype=y_local.dtype, device=y_local.device)
    padded[:, :y_local.shape[1]] = y_local
    full = torch.empty((world, rows, wmax), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(full.view(-1), padded.view(-1), group=group)
    return torch.cat([full[r, :, :c1 - c0] for r, (c0, c1) in enumerate(spans)], dim=1)


class TPLinear(torch.nn.Module):
    """A linear layer sharded by output tile: local forward on this rank's columns, then an
    all-gather.  `local` is this rank's module (an EXL3Linear built from shard_layer)."""

    def __init__(self, local: Callable[[torch.Tensor], torch.Tensor], out_features: int, group=None):
        super().__init__()
        self.__dict__["local"] = local
        self.out_features = out_features
        self.group = group

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        y = self.local(x.reshape(-1, x.shape[-1]))
        return all_gather_columns(y, self.out_features, self.group).reshape(lead + (self.out_features,))


# ---- expert parallel ---------------------------------------------------------------------------

def shard_experts(num_experts: int, world: int, rank: int) -> tuple[int, int]:
    """Expert range [e0, e1) of `rank`."""
    return shard_blocks(num_experts, world, rank)


def shard_expert_weights(w: dict, num_experts: int, world: int, rank: int) -> dict:
    """Slice stacked expert tensors (numpy or torch) to this rank's experts.  The stacked
    gate/up trellis holds all gates, then all ups, so the shard is two column ranges."""
    e0, e1 = shard_experts(num_experts, world, rank)
    gu = w["gu_trellis"]
    gt = gu.shape[1] // (2 * num_experts)
    dt = w["dn_trellis"].shape[1] // num_experts
    cat = np.concatenate if isinstance(gu, np.ndarray) else (lambda xs, axis: torch.cat(xs, dim=axis))
    return dict(
        gu_trellis=cat([gu[:, e0 * gt:e1 * gt], gu[:, (num_experts + e0) * gt:(num_experts + e1) * gt]], 1),
        gu_suh=w["gu_suh"][e0:e1], gu_svh=w["gu_svh"][e0:e1],
        dn_trellis=w["dn_trellis"][:, e0 * dt:e1 * dt], dn_suh=w["dn_suh"][e0:e1], dn_svh=w["dn_svh"][e0:e1])


class EPSwitchGLU(torch.nn.Module):
    """Stacked experts sharded by expert.  `local(x (1,T,D), idx (1,T,k)) -> (1,T,k,D)` is this
    rank's switch over its own experts (local indices).  `forward`: tokens replicated on every
    rank, pairs routed to another rank's expert are computed there, the partial outputs are
    summed.  `forward_partitioned`: many tokens, partitioned over the ranks."""

    def __init__(self, local: Callable, num_experts: int, group=None):
        super().__init__()
        self.__dict__["local"] = local
        self.num_experts = num_experts
        self.group = group

    def forward(self, x: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
        world, rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        e0, e1 = shard_experts(self.num_experts, world, rank)
        B, S, kk = indices.shape
        D = x.shape[-1]
        flat = indices.reshape(-1)
        ranged = getattr(self.local, "decode_range", None)
        if ranged is not None and x.is_cuda and B * S <= 16:
            # The library picks this rank's pairs on the device (a table of which only the first
            # entries are in use, their number never seen by the host): nothing here depends on
            # the routing, so the call — the all-reduce included — can be captured in a CUDA graph.
            out = ranged(x.reshape(B * S, D), indices.reshape(B * S, kk), (e0, e1, self.num_experts))
            out = out.reshape(B * S * kk, D)
            dist.all_reduce(out, group=self.group)
            return out.reshape(B, S, kk, D)
        mine = (flat >= e0) & (flat < e1)
        out = torch.zeros((B * S * kk, D), dtype=torch.float16, device=x.device)
        sel = torch.nonzero(mine).reshape(-1)                 # pairs this rank computes
        if sel.numel() > 0:
            tok = torch.div(sel, kk, rounding_mode="floor")
            xs = x.reshape(B * S, D)[tok]
            # every selected pair becomes a one-slot token for the local switch
            y = self.local(xs.reshape(1, -1, D), (flat[sel] - e0).reshape(1, -1, 1))
            out[sel] = y.reshape(-1, D).to(torch.float16)
        # each pair is written by exactly one rank and is zero elsewhere, so the fp16 sum is exact
        if out.device.type == "cpu":      # gloo has no fp16 reduction
            out32 = out.float()
            dist.all_reduce(out32, group=self.group)
            out = out32.to(torch.float16)
        else:
            dist.all_reduce(out, group=self.group)
        return out.reshape(B, S, kk, D)


    def forward_partitioned(self, x_local: torch.Tensor, idx_local: torch.Tensor) -> torch.Tensor:
        """Many tokens, partitioned over the ranks (T_local each, the same on every rank): all
        ranks gather the tokens and their routing (NCCL all-gather), every rank runs its experts
        over the pairs routed to them — picked and counted on the device — and its down
        projection stores each output row straight into the memory of the rank that owns the
        token (peer stores over NVLink, `exl3_gemm_tiles_peers`).  Returns this rank's
        (T_local, k, D) outputs, a view of an exchange buffer that the next call but two reuses.
        No value ever reaches the host, so the call can be captured in a CUDA graph (the exchange
        buffers rotate per call: a replayed graph must not run twice in a row, see PeerExchange)."""
        from . import _lib, ops

        world, rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        e0, e1 = shard_experts(self.num_experts, world, rank)
        T, kk = idx_local.shape
        D = x_local.shape[-1]
        n_local = T * kk
        ex = self.__dict__.get("_exchange")
        if ex is None or ex.max_rows < n_local or ex.max_cols != D:
            ex = PeerExchange(n_local, D, self.group, ring=3)
            self.__dict__["_exchange"] = ex
        x_all = torch.empty((world * T, D), dtype=x_local.dtype, device=x_local.device)
        dist.all_gather_into_tensor(x_all, x_local.contiguous(), group=self.group)
        idx_all = torch.empty((world * T, kk), dtype=idx_local.dtype, device=idx_local.device)
        dist.all_gather_into_tensor(idx_all, idx_local.contiguous(), group=self.group)
        _, y_ptrs, c_ptrs, view, my_ctr = ex.take(n_local, D)
        self.local.prefill_range(x_all, idx_all, (e0, e1, self.num_experts), (y_ptrs, c_ptrs, world, n_local, D))
        dev = x_local.device
        ws = ops.Workspace.get(dev, 1, 128)
        _lib.check(_lib.load().exl3_peer_wait(my_ctr, world, ws.buf.data_ptr(), 0,
                                              torch.cuda.current_stream(dev).cuda_stream), "exl3_peer_wait")
        return view.view(T, kk, D)


def dispatch_rows_to_experts(x_local: torch.Tensor, idx_local: torch.Tensor, num_experts: int, group=None):
    """Prefill exchange, step 1: tokens are partitioned over the ranks; every (token, slot) row
    goes to the rank that owns its expert.  Returns (rows received, their local expert index,
    the bookkeeping needed by return_rows_to_tokens)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    T, kk = idx_local.shape
    flat = idx_local.reshape(-1)
    bounds = torch.tensor([shard_experts(num_experts, world, r)[1] for r in range(world)],
                          device=flat.device)
    owner = torch.searchsorted(bounds, flat, right=True)
    order = torch.argsort(owner, stable=True)
    send_counts = torch.bincount(owner, minlength=world)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    sc, rc = send_counts.cpu().tolist(), recv_counts.cpu().tolist()
    rows = x_local[torch.div(order, kk, rounding_mode="floor")].contiguous()
    recv = torch.empty((sum(rc), x_local.shape[1]), dtype=x_local.dtype, device=x_local.device)
    dist.all_to_all_single(recv, rows, output_split_sizes=rc, input_split_sizes=sc, group=group)
    e_send = flat[order].contiguous()
    e_recv = torch.empty((sum(rc),), dtype=e_send.dtype, device=e_send.device)
    dist.all_to_all_single(e_recv, e_send, output_split_sizes=rc, input_split_sizes=sc, group=group)
    e0 = shard_experts(num_experts, world, rank)[0]
    return recv, e_recv - e0, (order, sc, rc, T, kk)


def return_rows_to_tokens(y_rows: torch.Tensor, book, group=None) -> torch.Tensor:
    """Prefill exchange, step 2: expert outputs travel back to the rank that owns the token;
    returns (T_local, k, D) in the original (token, slot) order."""
    order, sc, rc, T, kk = book
    back = torch.empty((sum(sc), y_rows.shape[1]), dtype=y_rows.dtype, device=y_rows.device)
    dist.all_to_all_single(back, y_rows.contiguous(), output_split_sizes=sc, input_split_sizes=rc,
                           group=group)
    out = torch.empty_like(back)
    out[order] = back
    return out.reshape(T, kk, -1)


# ---- output exchange over peer memory ----------------------------------------------------------

class PeerExchange:
    """Full-row buffers and arrival counters of all ranks, mapped into every process
    (torch symmetric memory: CUDA virtual-memory handles exchanged over the process group), for
    the library's peer-store all-gather (`exl3_gemv_peers`, `exl3_peer_allgather`,
    `exl3_peer_wait`).

    `ring` (buffer, counter) pairs are used in rotation; two CONSECUTIVE exchanges must not share
    a pair (a fast rank may send exchange j+1 while a slow one still reads j), so a caller that
    replays a fixed sequence of G exchanges (a captured step) needs (G - 1) % ring != 0 — see
    `ring_for`."""

    def __init__(self, max_rows: int, max_cols: int, group=None, ring: int = 4):
        import ctypes

        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("at most 8 peers")
        self.ring, self.max_rows, self.max_cols = ring, max_rows, max_cols
        dev = torch.device("cuda", torch.cuda.current_device())
        self.slot_elems = max_rows * max_cols
        # one allocation: the row buffers of the ring, then the counters (256 B apart)
        self._ctr_off = (ring * self.slot_elems * 2 + 255) // 256 * 256
        nbytes = self._ctr_off + ring * 256
        self.buf = symm.empty(nbytes, dtype=torch.uint8, device=dev)
        self.buf.zero_()
        torch.cuda.synchronize()
        self.handle = symm.rendezvous(self.buf, self.group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        dist.barrier(self.group)                      # everybody's counters are zero before first use
        self._u64 = ctypes.c_uint64 * self.world
        self._next = 0
        self.pending = None       # counter address of an exchange whose arrivals nobody has waited for yet

    @staticmethod
    def ring_for(exchanges_per_replay: int) -> int:
        """Smallest ring >= 3 whose rotation never puts the last exchange of a replayed sequence and
        the first of the next replay on the same pair."""
        if exchanges_per_replay < 2:
            raise ValueError("a replayed sequence needs at least two exchanges: with one, every replay "
                             "would land on the same pair back to back")
        r = 3
        while (exchanges_per_replay - 1) % r == 0:
            r += 1
        return r

    def settle(self, pdl: bool = False) -> None:
        """Launch the wait for a pending exchange (see ops.gemv_peers, defer_wait): after it, this
        rank's row of that exchange is complete for every later kernel of the stream."""
        if self.pending is None:
            return
        from . import _lib, ops

        dev = torch.device("cuda", torch.cuda.current_device())
        ws = ops.Workspace.get(dev, 1, 128)
        _lib.check(_lib.load().exl3_peer_wait(self.pending, self.world, ws.buf.data_ptr(),
                                              _lib.FLAG_PDL if pdl else 0,
                                              torch.cuda.current_stream(dev).cuda_stream), "exl3_peer_wait")
        self.pending = None

    def restart(self) -> None:
        """Start the rotation over: call at the top of a sequence that is captured in a CUDA graph
        and replayed, so that every replay (and the eager run before the capture) walks the same
        pairs.  Purely eager callers need not restart at all."""
        self._next = 0

    def take(self, rows: int, cols: int):
        """Next pair of the ring: (slot index, host arrays of all ranks' buffer and counter pointers,
        this rank's (rows, cols) view of its buffer, this rank's counter address)."""
        if rows > self.max_rows or rows * cols > self.slot_elems:
            raise ValueError("exchange larger than the ring's slots")
        s = self._next
        self._next = (s + 1) % self.ring
        y = self._u64(*[p + s * self.slot_elems * 2 for p in self.ptrs])
        c = self._u64(*[p + self._ctr_off + s * 256 for p in self.ptrs])
        base = s * self.slot_elems * 2
        view = self.buf[base:base + rows * cols * 2].view(torch.float16).view(rows, cols)
        return s, y, c, view, self.ptrs[self.rank] + self._ctr_off + s * 256
