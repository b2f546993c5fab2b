"""Host-side logic of the multi-GPU paths on CPU: world_size 2 and 3 `gloo` ranks, with the
CPU oracle standing in for each rank's local kernel (the oracle is the checker here too: the
sharded result must equal the unsharded one)."""

from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(fn, world, *args):
    port = _free_port()
    mp.spawn(_entry, args=(world, port, fn, args), nprocs=world, join=True)


def _entry(rank, world, port, fn, args):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        fn(rank, world, *args)
    finally:
        dist.destroy_process_group()


def test_shard_ranges_cover_everything_once():
    from ponyexl3_b200.parallel import shard_blocks, shard_columns, shard_experts

    for n in (1, 7, 40, 136, 1187):
        for world in (1, 2, 3, 4, 8):
            got = [shard_blocks(n, world, r) for r in range(world)]
            assert got[0][0] == 0 and got[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
            sizes = [b - a for a, b in got]
            assert max(sizes) - min(sizes) <= 1
    assert shard_columns(151936, 8, 0) == (0, 149 * 128)        # 1187 blocks: 149,149,149,148,...
    assert shard_columns(151936, 8, 7)[1] == 151936
    assert shard_experts(256, 8, 3) == (96, 128)
    with pytest.raises(ValueError):
        shard_columns(100, 2, 0)
    with pytest.raises(ValueError):
        shard_blocks(8, 2, 2)


def test_peer_exchange_ring_never_reuses_a_pair_back_to_back():
    """A replayed sequence of G exchanges over a ring of R pairs uses pair j % R; the last exchange
    of one replay and the first of the next must differ, like any two neighbours."""
    from ponyexl3_b200.parallel import PeerExchange

    for g in list(range(2, 40)) + [48, 256, 257, 258]:
        r = PeerExchange.ring_for(g)
        assert r >= 3
        seq = [j % r for j in range(g)] * 3                  # three replays back to back
        assert all(a != b for a, b in zip(seq, seq[1:])), (g, r)
    with pytest.raises(ValueError):
        PeerExchange.ring_for(1)


def _tp_worker(rank, world, outf):
    from conftest import synthetic_layer
    from oracle import exl3_oracle as oracle
    from ponyexl3_b200 import EXL3Layer
    from ponyexl3_b200.parallel import TPLinear, shard_layer

    k, inf = 4, 256
    tr, suh, svh, bias = synthetic_layer(k, inf, outf, 123, bias=True)
    layer = EXL3Layer("tp", inf, outf, k, tr, suh, svh, bias)
    shard = shard_layer(layer, world, rank)
    shard.validate()

    def local(x2d):
        if shard.out_features == 0:
            return torch.empty((x2d.shape[0], 0), dtype=torch.float16)
        y = oracle.linear_forward(x2d.numpy(), shard.trellis, k, 0, shard.suh, shard.svh, shard.bias)
        return torch.from_numpy(y)

    x = np.random.default_rng(1).standard_normal((2, 3, inf)).astype(np.float16)
    y = TPLinear(local, outf)(torch.from_numpy(x))
    want = oracle.linear_forward(x, tr, k, 0, suh, svh, bias)
    assert y.shape == (2, 3, outf)
    assert np.array_equal(y.numpy().view(np.uint16), want.view(np.uint16)), f"rank {rank}"


@pytest.mark.parametrize("world,outf", [(2, 512), (3, 512), (2, 384)])
def test_tensor_parallel_by_output_tile_equals_unsharded(world, outf):
    _run(_tp_worker, world, outf)


def _experts(E, D, H, k, seed):
    rng = np.random.default_rng(seed)
    sg = lambda *s: np.where(rng.random(s) > 0.5, -1.0, 1.0).astype(np.float16)
    return dict(gu_trellis=rng.integers(0, 65536, size=(D // 16, E * 2 * H // 16, 16 * k), dtype=np.uint16),
                gu_suh=sg(E, 2, D), gu_svh=sg(E, 2 * H),
                dn_trellis=rng.integers(0, 65536, size=(H // 16, E * D // 16, 16 * k), dtype=np.uint16),
                dn_suh=sg(E, H), dn_svh=sg(E, D))


def _ep_worker(rank, world):
    from oracle import exl3_oracle as oracle
    from ponyexl3_b200.parallel import (EPSwitchGLU, dispatch_rows_to_experts, return_rows_to_tokens,
                                        shard_expert_weights, shard_experts)

    E, D, H, kk, k = 6, 128, 128, 2, 4
    w = _experts(E, D, H, k, 9)
    mine = shard_expert_weights(w, E, world, rank)
    e0, e1 = shard_experts(E, world, rank)

    def local(x, idx):
        y = oracle.switch_glu(x.reshape(-1, D).numpy(), idx.reshape(-1, idx.shape[-1]).numpy(), **mine,
                              k=k, cb=0)
        return torch.from_numpy(y).reshape(1, -1, idx.shape[-1], D)

    rng = np.random.default_rng(3)
    T = 5
    x = (rng.standard_normal((T, D)) * 0.5).astype(np.float16)
    idx = np.stack([rng.choice(E, size=kk, replace=False) for _ in range(T)]).astype(np.int64)
    want = oracle.switch_glu(x, idx, **w, k=k, cb=0)

    # decode-class: replicated tokens, partial outputs summed
    y = EPSwitchGLU(local, E)(torch.from_numpy(x).view(1, T, D), torch.from_numpy(idx).view(1, T, kk))
    assert np.array_equal(y.numpy().reshape(T, kk, D).view(np.uint16), want.view(np.uint16))

    # prefill-class: tokens partitioned over the ranks, rows exchanged with all-to-all
    t0, t1 = T * rank // world, T * (rank + 1) // world
    xl, il = torch.from_numpy(x[t0:t1]), torch.from_numpy(idx[t0:t1])
    rows, e_local, book = dispatch_rows_to_experts(xl, il, E)
    assert ((e_local >= 0) & (e_local < e1 - e0)).all()
    if rows.shape[0]:
        yr = local(rows.reshape(1, -1, D), e_local.reshape(1, -1, 1)).reshape(-1, D)
    else:
        yr = torch.empty((0, D), dtype=torch.float16)
    back = return_rows_to_tokens(yr, book)
    assert np.array_equal(back.numpy().view(np.uint16), want[t0:t1].view(np.uint16))


@pytest.mark.parametrize("world", [2, 3])
def test_expert_parallel_equals_unsharded(world):
    _run(_ep_worker, world)
