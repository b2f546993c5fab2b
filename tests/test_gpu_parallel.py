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
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_two_gpus_equals_one():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)
