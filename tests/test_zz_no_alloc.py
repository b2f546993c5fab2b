"""exl3_gemv_noalloc — the GEMV for callers that cannot allocate device memory (plug-in hosts
that are only handed input and output buffers, decode loops where cudaMalloc is off limits).
Its scratch is a fixed array inside the library, so the call takes no workspace.

Called here through the C ABI and compared with exl3_gemv and with the CPU oracle on the same
inputs, several calls in a row with different shapes (each finds the array holding the previous
call's data); the status word of the built-in scratch must stay 0.
The file name sorts last so that every other test has run before this one in a `-x` run.
"""

from __future__ import annotations

import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

REL_TOL = 1e-3


def _call_pair(lib, ops, oracle, rows, inf, outf, k, cb, seed):
    dev = torch.device("cuda")
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    tr = torch.randint(-32768, 32767, (inf // 16, outf // 16, 16 * k), dtype=torch.int16, device=dev,
                       generator=g)
    suh = (torch.randint(0, 2, (inf,), device=dev, generator=g) * 2 - 1).to(torch.float16)
    svh = (torch.randint(0, 2, (outf,), device=dev, generator=g) * 2 - 1).to(torch.float16)
    bias = (torch.randn(outf, device=dev, generator=g) * 0.01).to(torch.float16)
    x = torch.randn((rows, inf), device=dev, generator=g).to(torch.float16)
    want = ops.gemv(x, tr, k, cb, suh, svh, bias)                 # existing entry point
    got = torch.full_like(want, float("nan"))
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.exl3_gemv_noalloc(x.data_ptr(), 0, rows, x.stride(0), tr.data_ptr(), inf // 16,
                               outf // 16, k, cb, suh.data_ptr(), svh.data_ptr(), bias.data_ptr(),
                               got.data_ptr(), got.stride(0), 0, stream)
    assert rc == 0, lib.exl3_error_string(rc)
    torch.cuda.synchronize()
    ref = oracle.linear_forward(x.cpu().numpy(), tr.cpu().numpy().view(np.uint16), k, cb, suh.cpu().numpy(),
                                svh.cpu().numpy(), bias.cpu().numpy())
    return got, want, torch.from_numpy(ref.astype(np.float32))


def test_noalloc_matches_workspace_entry_point_twice_in_a_row(oracle):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from ponyexl3_b200 import _lib, ops

    lib = _lib.load()
    # first call: 12 rows -> the rotated activations go through the built-in scratch
    # second call: other shape and K, fewer rows -> the array still holds the first call's words
    for rows, inf, outf, k, cb, seed in ((12, 2048, 1024, 4, 0, 1), (5, 4096, 512, 5, 1, 2),
                                         (1, 5120, 5120, 4, 0, 3)):
        got, want, ref = _call_pair(lib, ops, oracle, rows, inf, outf, k, cb, seed)
        assert torch.isfinite(got.float()).all()
        err = float((got.float() - want.float()).norm() / want.float().norm())
        assert err <= REL_TOL, f"rows={rows}: rel err {err} against exl3_gemv"
        err = float((got.float().cpu() - ref).norm() / ref.norm())
        assert err <= REL_TOL, f"rows={rows}: rel err {err} against the oracle"
    status = ctypes.c_int(-1)
    assert lib.exl3_gemv_noalloc_status(ctypes.byref(status), torch.cuda.current_stream().cuda_stream) == 0
    assert status.value == 0


def test_noalloc_rejects_sizes_beyond_its_scratch():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from ponyexl3_b200 import _lib

    lib = _lib.load()
    buf = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    # 16 rows x 32,768 features = 524,288 elements > 262,144: refused before any launch
    rc = lib.exl3_gemv_noalloc(p, 0, 16, 32768, p, 2048, 8, 4, 0, None, None, None, p, 128, 0, None)
    assert rc == -10
    assert b"range" in lib.exl3_error_string(rc)
    assert lib.exl3_gemv_noalloc(p, 0, 17, 128, p, 8, 8, 4, 0, None, None, None, p, 128, 0, None) == -5
