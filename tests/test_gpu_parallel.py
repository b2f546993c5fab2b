"""Two-GPU check of the sharded paths with the real kernels (skipped on a single-GPU box):
tensor parallel by output tile + NCCL all-gather, and expert parallel + all-reduce, must equal
the unsharded module on one GPU."""

from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port):
    import torch.distributed as dist
    from conftest import synthetic_layer
    from ponyexl3_b200 import EXL3Layer
    from ponyexl3_b200.linear import EXL3Linear
    from ponyexl3_b200.parallel import TPLinear, shard_layer

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        for outf in (1024, 384):           # even and uneven block split
            tr, suh, svh, bias = synthetic_layer(4, 2048, outf, 321, bias=True)
            layer = EXL3Layer("tp", 2048, outf, 4, tr, suh, svh, bias)
            x = torch.from_numpy(np.random.default_rng(2).standard_normal((3, 2048)).astype(np.float16)).cuda()
            full = EXL3Linear(layer, device=f"cuda:{rank}")(x)
            shard = shard_layer(layer, world, rank)
            y = TPLinear(EXL3Linear(shard, device=f"cuda:{rank}"), outf)(x)
            assert torch.equal(y, full), f"rank {rank} outf {outf}"
        _expert_parallel(rank, world)
        _dense_step(rank, world)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _expert_parallel(rank, world):
    """Experts sharded by expert: replicated-token decode path (all-reduce) and partitioned-token
    prefill path (two all-to-alls) against the unsharded switch on the same GPU."""
    from ponyexl3_b200.moe import EXL3SwitchGLU
    from ponyexl3_b200.parallel import (EPSwitchGLU, dispatch_rows_to_experts, return_rows_to_tokens,
                                        shard_expert_weights, shard_experts)
    dev = torch.device("cuda", rank)
    E, D, H, kk, k = 8, 256, 128, 2, 4
    g = torch.Generator(device=dev)
    g.manual_seed(77)                                   # same draw on both ranks
    sg = lambda *s: (torch.randint(0, 2, s, device=dev, generator=g) * 2 - 1).to(torch.float16)
    w = dict(gu_trellis=torch.randint(-32768, 32767, (D // 16, E * 2 * H // 16, 16 * k), dtype=torch.int16,
                                      device=dev, generator=g),
             gu_suh=sg(E, 2, D), gu_svh=sg(E, 2 * H) * 0.05,
             dn_trellis=torch.randint(-32768, 32767, (H // 16, E * D // 16, 16 * k), dtype=torch.int16,
                                      device=dev, generator=g),
             dn_suh=sg(E, H), dn_svh=sg(E, D) * 0.05)
    full = EXL3SwitchGLU(**w, k=k, cb=0)
    local = EXL3SwitchGLU(**shard_expert_weights(w, E, world, rank), k=k, cb=0)
    T = 6
    x = (torch.randn((T, D), device=dev, generator=g) * 0.5).to(torch.float16)
    idx = torch.stack([torch.randperm(E, device=dev, generator=g)[:kk] for _ in range(T)])
    want = full(x.view(1, T, D), idx.view(1, T, kk)).reshape(T, kk, D)
    got = EPSwitchGLU(local, E)(x.view(1, T, D), idx.view(1, T, kk)).reshape(T, kk, D)
    assert torch.equal(got, want), f"rank {rank}: expert-parallel decode path"
    t0, t1 = T * rank // world, T * (rank + 1) // world
    rows, e_local, book = dispatch_rows_to_experts(x[t0:t1].contiguous(), idx[t0:t1].contiguous(), E)
    e0, e1 = shard_experts(E, world, rank)
    assert bool(((e_local >= 0) & (e_local < e1 - e0)).all())
    if rows.shape[0]:
        yr = local(rows.reshape(1, -1, D), e_local.reshape(1, -1, 1)).reshape(-1, D)
    else:
        yr = torch.empty((0, D), dtype=torch.float16, device=dev)
    back = return_rows_to_tokens(yr, book)
    assert torch.equal(back, want[t0:t1]), f"rank {rank}: expert-parallel exchange path"
    # many tokens, partitioned: gathered tokens, pairs picked on the device, rows stored into the
    # owner's memory over the peer mapping; twice, so that the exchange buffers rotate
    T2 = 64
    x2 = (torch.randn((T2, D), device=dev, generator=g) * 0.5).to(torch.float16)
    idx2 = torch.stack([torch.randperm(E, device=dev, generator=g)[:kk] for _ in range(T2)])
    want2 = full(x2.view(1, T2, D), idx2.view(1, T2, kk)).reshape(T2, kk, D)
    a0, a1 = T2 * rank // world, T2 * (rank + 1) // world
    ep = EPSwitchGLU(local, E)
    for rep in range(2):
        got2 = ep.forward_partitioned(x2[a0:a1].contiguous(), idx2[a0:a1].contiguous())
        torch.cuda.synchronize()
        assert torch.equal(got2, want2[a0:a1]), f"rank {rank}: expert-parallel partitioned path, call {rep}"
    from ponyexl3_b200 import ops
    assert ops.Workspace.get(dev, 1, 128).status() == 0


def _dense_step(rank, world):
    """The tensor-parallel decode step picks the same tokens as the same model on one GPU."""
    from ponyexl3_b200.dense_step import DenseConfig, SyntheticDenseDecoder
    dev = torch.device("cuda", rank)
    cfg = DenseConfig(layers=2, hidden=512, intermediate=768, q_heads=4, kv_heads=2, head_dim=128,
                      vocab=1152, context=40, max_rows=4)
    one = SyntheticDenseDecoder(cfg, dev, seed=21, tensor_parallel=False)
    tp = SyntheticDenseDecoder(cfg, dev, seed=21)                        # exchanges over peer memory
    tp_nccl = SyntheticDenseDecoder(cfg, dev, seed=21, peer_exchange=False)
    assert tp.world == world and one.world == 1 and tp.peer is not None and tp_nccl.peer is None
    for rows in (1, 3):
        tok = torch.tensor([3, 700, 41][:rows], device=dev)
        want = one.forward_logits(tok).float()
        v0, v1 = tp.vocab_span
        for name, m in (("peer", tp), ("nccl", tp_nccl)):
            got = m.forward_logits(tok).float()
            err = (got - want[:, v0:v1]).norm() / want[:, v0:v1].norm()
            assert float(err) < 2e-3, f"rank {rank} rows {rows} {name}: {float(err)}"
            assert torch.equal(m.step(tok), one.step(tok))
    # many steps back to back: the ring of buffers and counters keeps the ranks apart
    tok = torch.tensor([5], device=dev)
    ref = tp_nccl.step(tok)
    for _ in range(20):
        assert torch.equal(tp.step(tok), ref)
    from ponyexl3_b200 import ops
    assert ops.Workspace.get(dev, 1, 128).status() == 0


def test_tensor_parallel_two_gpus_equals_one():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)
