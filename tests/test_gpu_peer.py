"""The peer-store output exchange on ONE GPU: with a single "peer" (this GPU's own buffers) the
fused epilogue, the copy kernel and the bounded wait can be checked without a second device.
The two-GPU run is in test_gpu_parallel.py."""

import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _u64(*vals):
    return (ctypes.c_uint64 * len(vals))(*vals)


@pytest.fixture(scope="module")
def lib():
    from ponyexl3_b200 import _lib
    return _lib.load()


def _private_ws():
    from ponyexl3_b200 import _lib
    lib = _lib.load()
    n = int(lib.exl3_workspace_bytes(16, 32768))
    ws = torch.zeros(n, dtype=torch.uint8, device="cuda")
    return ws, n


def _status(lib, ws):
    out = ctypes.c_int(0)
    assert lib.exl3_workspace_status(ws.data_ptr(), ctypes.byref(out), torch.cuda.current_stream().cuda_stream) == 0
    return out.value


@pytest.mark.parametrize("rows,k", [(1, 4), (5, 4), (16, 5)])
def test_gemv_peers_single_peer_equals_gemv(lib, rows, k):
    from ponyexl3_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(6)
    inf, outf, col0, full = 1024, 768, 256, 1536              # a slice placed inside a wider row
    tr = torch.randint(-32768, 32767, (inf // 16, outf // 16, 16 * k), dtype=torch.int16, device="cuda", generator=g)
    suh = (torch.randint(0, 2, (inf,), device="cuda", generator=g) * 2 - 1).half()
    svh = (torch.randint(0, 2, (outf,), device="cuda", generator=g) * 2 - 1).half() * 0.03
    x = torch.randn((rows, inf), device="cuda", generator=g).half()
    want = ops.gemv(x, tr, k, 0, suh, svh, None)
    ws, n = _private_ws()
    y_full = torch.full((rows, full), 7.0, dtype=torch.float16, device="cuda")
    ctr = torch.zeros(64, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    rc = lib.exl3_gemv_peers(x.data_ptr(), 0, rows, x.stride(0), tr.data_ptr(), inf // 16, outf // 16, k, 0,
                             suh.data_ptr(), svh.data_ptr(), None, _u64(y_full.data_ptr()), _u64(ctr.data_ptr()),
                             1, full, col0, ws.data_ptr(), n, 0, st)
    assert rc == 0
    assert lib.exl3_peer_wait(ctr.data_ptr(), 1, ws.data_ptr(), 0, st) == 0
    torch.cuda.synchronize()
    assert _status(lib, ws) == 0
    assert int(ctr[0]) == 0                                     # re-armed by the waiter
    assert torch.equal(y_full[:, col0:col0 + outf], want)
    assert bool((y_full[:, :col0] == 7).all()) and bool((y_full[:, col0 + outf:] == 7).all())


def test_peer_allgather_single_peer(lib):
    g = torch.Generator(device="cuda").manual_seed(7)
    rows, cols, full, col0 = 3, 640, 2048, 1024
    src = torch.randn((rows, cols), device="cuda", generator=g).half()
    dst = torch.zeros((rows, full), dtype=torch.float16, device="cuda")
    ctr = torch.zeros(64, dtype=torch.int32, device="cuda")
    ws, _ = _private_ws()
    st = torch.cuda.current_stream().cuda_stream
    assert lib.exl3_peer_allgather(src.data_ptr(), rows, cols, src.stride(0), _u64(dst.data_ptr()),
                                   _u64(ctr.data_ptr()), 1, full, col0, 0, st) == 0
    assert lib.exl3_peer_wait(ctr.data_ptr(), 1, ws.data_ptr(), 0, st) == 0
    torch.cuda.synchronize()
    assert _status(lib, ws) == 0 and int(ctr[0]) == 0
    assert torch.equal(dst[:, col0:col0 + cols], src) and float(dst[:, :col0].abs().sum()) == 0


def test_peer_wait_gives_up_and_reports(lib):
    """A counter nobody increments: the poll ends by itself after about a second with the
    peer-timeout bit in the status word; the context stays usable."""
    import time
    ctr = torch.zeros(64, dtype=torch.int32, device="cuda")
    ws, _ = _private_ws()
    st = torch.cuda.current_stream().cuda_stream
    t0 = time.perf_counter()
    assert lib.exl3_peer_wait(ctr.data_ptr(), 1, ws.data_ptr(), 0, st) == 0
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert _status(lib, ws) & 16
    assert dt < 10.0
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0


def test_peer_entry_points_validate(lib):
    ws, n = _private_ws()
    st = torch.cuda.current_stream().cuda_stream
    ctr = torch.zeros(4, dtype=torch.int32, device="cuda")
    assert lib.exl3_peer_wait(None, 1, ws.data_ptr(), 0, st) == -1            # EXL3_E_NULL
    assert lib.exl3_peer_wait(ctr.data_ptr(), 0, ws.data_ptr(), 0, st) != 0   # zero arrivals make no sense
    src = torch.zeros((1, 64), dtype=torch.float16, device="cuda")
    assert lib.exl3_peer_allgather(src.data_ptr(), 1, 64, 64, _u64(src.data_ptr()), _u64(ctr.data_ptr()), 9, 64, 0,
                                   0, st) != 0                               # more than 8 peers
