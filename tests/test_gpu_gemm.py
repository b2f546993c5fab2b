"""GPU parity of the tensor-core prefill GEMM (rows > 16) through the module and the C ABI,
against the CPU oracle.  Tolerance: relative L2 error <= 1e-3 (fp32 accumulate)."""

from __future__ import annotations

import numpy as np
import pytest

from conftest import rel_err, synthetic_layer

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

REL_TOL = 1e-3


@pytest.fixture(scope="module")
def mod():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import ponyexl3_b200
    from ponyexl3_b200 import ops
    from ponyexl3_b200.linear import EXL3Linear

    class NS:
        pass

    ns = NS()
    ns.ops, ns.EXL3Linear, ns.EXL3Layer = ops, EXL3Linear, ponyexl3_b200.EXL3Layer
    return ns


def _layer(mod, k, inf, outf, seed, cb=0, bias=False):
    tr, suh, svh, b = synthetic_layer(k, inf, outf, seed, bias=bias)
    return mod.EXL3Layer("test", inf, outf, k, tr, suh, svh, b, mcg=(cb == 1), mul1=(cb == 2))


def _check(mod, oracle, layer, x):
    m = mod.EXL3Linear(layer)
    y = m(torch.from_numpy(x).cuda()).cpu().numpy()
    want = oracle.linear_forward(x.astype(np.float16), layer.trellis, layer.k, layer.codebook_mode,
                                 layer.suh, layer.svh, layer.bias)
    assert y.shape == want.shape and y.dtype == np.float16
    assert np.isfinite(y.astype(np.float32)).all()
    e = rel_err(y, want)
    assert e <= REL_TOL, f"rel err {e}"
    assert mod.ops.Workspace.get(torch.device("cuda"), 1, 128).status() == 0


@pytest.mark.parametrize("k", range(1, 9))
@pytest.mark.parametrize("cb", [0, 1, 2])
def test_gemm_all_k_all_codebooks(mod, oracle, k, cb):
    layer = _layer(mod, k, 256, 384, seed=500 + 10 * k + cb, cb=cb, bias=(k % 2 == 1))
    x = np.random.default_rng(k).standard_normal((40, 256)).astype(np.float16)
    _check(mod, oracle, layer, x)


@pytest.mark.parametrize("k,cb,bias", [(4, 0, False), (2, 1, True), (5, 2, False), (8, 0, True), (1, 0, False)])
@pytest.mark.parametrize("rows,inf,outf", [(1024, 256, 256), (1500, 512, 384), (2049, 128, 640)])
def test_gemm_on_cta_pairs(mod, oracle, rows, inf, outf, k, cb, bias):
    """The prefill GEMM on pairs of SMs (tcgen05.mma.cta_group::2, 512-row output tiles, each CTA
    decoding half of the B tile; selected through the tuning hook): whole and ragged row tiles, a
    last column tile of 128 columns, several tiles per pair, against the oracle; and the one-CTA
    kernel gives the same bits."""
    from ponyexl3_b200 import _lib

    layer = _layer(mod, k, inf, outf, seed=7000 + rows + k, cb=cb, bias=bias)
    x = np.random.default_rng(rows + k).standard_normal((rows, inf)).astype(np.float16)
    m = mod.EXL3Linear(layer)
    xd = torch.from_numpy(x).cuda()
    y_one = m(xd).clone()
    _lib.load().exl3_tune_gemm_pairs(1)
    try:
        _check(mod, oracle, layer, x)
        y_pair = m(xd).clone()
    finally:
        _lib.load().exl3_tune_gemm_pairs(0)
    assert torch.equal(y_pair, y_one)


@pytest.mark.parametrize("rows", [17, 128, 129, 256, 300, 513])
def test_gemm_ragged_row_counts(mod, oracle, rows):
    layer = _layer(mod, 4, 512, 256, seed=77)
    x = np.random.default_rng(rows).standard_normal((rows, 512)).astype(np.float16)
    _check(mod, oracle, layer, x)


def test_gemm_many_tiles_and_k_steps(mod, oracle):
    """More tiles than one wave of k-steps per stage ring, several tiles per CTA."""
    layer = _layer(mod, 4, 2048, 1280, seed=78, bias=True)
    x = np.random.default_rng(5).standard_normal((600, 2048)).astype(np.float16)
    _check(mod, oracle, layer, x)


def test_gemm_bf16_activations(mod, oracle):
    layer = _layer(mod, 4, 512, 512, seed=79)
    xb = torch.from_numpy(np.random.default_rng(6).standard_normal((200, 512)).astype(np.float32)).cuda().to(torch.bfloat16)
    y = mod.EXL3Linear(layer)(xb).cpu().numpy()
    want = oracle.linear_forward(xb.float().cpu().numpy().astype(np.float16), layer.trellis, 4, 0,
                                 layer.suh, layer.svh, None)
    assert rel_err(y, want) <= REL_TOL


def test_gemm_matches_gemv_rows(mod):
    """The two kernels implement one contract: the same rows through either agree."""
    layer = _layer(mod, 5, 1024, 768, seed=80, bias=True)
    m = mod.EXL3Linear(layer)
    x = torch.from_numpy(np.random.default_rng(7).standard_normal((64, 1024)).astype(np.float16)).cuda()
    big = m(x)
    small = torch.cat([m(x[i:i + 16]) for i in range(0, 64, 16)])
    assert (big.float() - small.float()).norm() / small.float().norm() < 5e-4


def test_config3_prefill_shape_sampled(mod, oracle):
    """M = 8192 tokens x 5120 -> 5120, K = 4, 3INST, bf16 activations: full run on the GPU,
    512 sampled rows checked against the oracle (the oracle's decode is shared)."""
    layer = _layer(mod, 4, 5120, 5120, seed=3000)
    rng = np.random.default_rng(3001)
    xb = torch.from_numpy(rng.standard_normal((8192, 5120)).astype(np.float32)).cuda().to(torch.bfloat16)
    y = mod.EXL3Linear(layer)(xb)
    assert mod.ops.Workspace.get(torch.device("cuda"), 1, 128).status() == 0
    idx = np.sort(rng.choice(8192, size=512, replace=False))
    xs = xb[torch.from_numpy(idx).cuda()].float().cpu().numpy().astype(np.float16)
    w = oracle.decode_packed_trellis(layer.trellis, 4, 0)
    want = oracle.linear_forward(xs, layer.trellis, 4, 0, layer.suh, layer.svh, None, w=w)
    assert rel_err(y[torch.from_numpy(idx).cuda()].cpu().numpy(), want) <= REL_TOL
