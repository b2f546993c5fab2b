"""GPU parity of the codec pieces, through the C ABI: bit-exact against the CPU
oracle and against the golden vectors made by the reference."""

from __future__ import annotations

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from ponyexl3_b200 import ops as _ops

    return _ops


def _dev(a: np.ndarray):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda()


@pytest.mark.parametrize("cb", [0, 1, 2])
def test_codebook_all_codewords_bit_exact(ops, oracle, cb):
    got = ops.codebook_table(cb).cpu().numpy().view(np.uint16)
    np.testing.assert_array_equal(got, oracle.codebook_table(cb).view(np.uint16))


@pytest.mark.parametrize("k", range(1, 9))
def test_unpack_bit_exact(ops, oracle, golden, k):
    g = golden["trellis"]
    got = ops.unpack_trellis(_dev(g[f"packed3_k{k}"]), k).cpu().numpy().view(np.uint16)
    np.testing.assert_array_equal(got, g[f"codewords3_k{k}"])
    rng = np.random.default_rng(k)
    packed = rng.integers(0, 65536, size=(7, 5, 16 * k), dtype=np.uint16)
    packed[0, 0] = 0xFFFF
    packed[0, 1] = 0
    got = ops.unpack_trellis(_dev(packed), k).cpu().numpy().view(np.uint16)
    np.testing.assert_array_equal(got, oracle.unpack_trellis(packed, k))


@pytest.mark.parametrize("k", range(1, 9))
@pytest.mark.parametrize("cb", [0, 1, 2])
def test_decode_bit_exact(ops, oracle, golden, k, cb):
    g = golden["tiles"]
    tile = ops.decode_packed_trellis(_dev(g[f"packed_k{k}_cb{cb}"].reshape(1, 1, -1)), k, cb)
    np.testing.assert_array_equal(tile.cpu().numpy().view(np.uint16), g[f"tile_k{k}_cb{cb}"])
    rng = np.random.default_rng(100 * k + cb)
    tr = rng.integers(0, 65536, size=(24, 16, 16 * k), dtype=np.uint16)
    w = ops.decode_packed_trellis(_dev(tr), k, cb).cpu().numpy()
    np.testing.assert_array_equal(w.view(np.uint16), oracle.decode_packed_trellis(tr, k, cb).view(np.uint16))
    sl = ops.decode_packed_trellis(_dev(tr), k, cb, n_offset=128, n_count=128).cpu().numpy()
    np.testing.assert_array_equal(sl.view(np.uint16), w[:, 128:].view(np.uint16))


def test_decode_config1_layer_bit_exact(ops, oracle):
    """in = out = 4096, K = 4, 3INST: all 16,777,216 weights."""
    rng = np.random.default_rng(1000)
    tr = rng.integers(0, 65536, size=(256, 256, 64), dtype=np.uint16)
    w = ops.decode_packed_trellis(_dev(tr), 4, 0).cpu().numpy()
    np.testing.assert_array_equal(w.view(np.uint16), oracle.decode_packed_trellis(tr, 4, 0).view(np.uint16))


def test_decode_errors(ops):
    tr = torch.zeros((3, 16, 64), dtype=torch.int16, device="cuda")
    with pytest.raises(ValueError):
        ops.decode_packed_trellis(tr, 3, 0)
    with pytest.raises(ValueError):
        ops.decode_packed_trellis(tr, 4, 0, n_offset=64)
    with pytest.raises(ValueError):
        ops.decode_packed_trellis(tr, 4, 0, n_offset=128, n_count=256)
    with pytest.raises(ValueError):
        ops.unpack_trellis(tr, 5)
    assert ops.unpack_trellis(tr[:0], 4).shape == (0, 16, 256)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16", "float32"])
def test_hadamard_matches_oracle(ops, oracle, golden, dtype):
    g = golden["hadamard"]
    x16 = g["x"].view(np.float16)
    pre, post = g["pre"].view(np.float16), g["post"].view(np.float16)
    xt = torch.from_numpy(x16.astype(np.float32)).cuda().to(getattr(torch, dtype))
    xin = xt.to(torch.float16).cpu().numpy()  # the values the kernel sees after its fp16 rounding
    for kw_np, kw_t in (({}, {}),
                        (dict(pre_scale=pre), dict(pre_scale=torch.from_numpy(pre).cuda())),
                        (dict(pre_scale=pre, post_scale=post),
                         dict(pre_scale=torch.from_numpy(pre).cuda(),
                              post_scale=torch.from_numpy(post).cuda()))):
        want = oracle.had_r_128(xin.astype(np.float32), **kw_np).astype(np.float16)
        got = ops.had_r_128(xt, **kw_t).cpu().numpy()
        # same math in a different float32 summation order: at most one fp16 ulp apart
        d = np.abs(got.view(np.int16).astype(np.int32) - want.view(np.int16).astype(np.int32))
        assert d.max() <= 1 and (d > 0).mean() < 0.01
    if dtype == "float16":
        want = g["y_both"].astype(np.float16)
        got = ops.had_r_128(xt, pre_scale=torch.from_numpy(pre).cuda(),
                            post_scale=torch.from_numpy(post).cuda()).cpu().numpy()
        d = np.abs(got.view(np.int16).astype(np.int32) - want.view(np.int16).astype(np.int32))
        assert d.max() <= 1


@pytest.mark.parametrize("dtype", ["float16", "bfloat16", "float32"])
@pytest.mark.parametrize("rows,n", [(64, 128), (200, 384), (1031, 256)])
def test_hadamard_of_many_rows_on_the_tensor_cores(ops, oracle, dtype, rows, n):
    """From 64 rows on the rotation runs as 16-row blocks of mma products with the +-1 matrix
    (whole and ragged row blocks, with and without the input scale); same values as the oracle
    up to the float32 summation order: at most one fp16 ulp apart, and rarely."""
    rng = np.random.default_rng(rows + n)
    x = rng.standard_normal((rows, n)).astype(np.float32)
    pre = np.where(rng.random(n) > 0.5, -1.0, 1.0).astype(np.float16)
    xt = torch.from_numpy(x).cuda().to(getattr(torch, dtype))
    xin = xt.to(torch.float16).cpu().numpy()
    for kw_np, kw_t in (({}, {}), (dict(pre_scale=pre), dict(pre_scale=torch.from_numpy(pre).cuda()))):
        want = oracle.had_r_128(xin.astype(np.float32), **kw_np).astype(np.float16)
        got = ops.had_r_128(xt, **kw_t).cpu().numpy()
        d = np.abs(got.view(np.int16).astype(np.int32) - want.view(np.int16).astype(np.int32))
        assert d.max() <= 1 and (d > 0).mean() < 0.01


def test_hadamard_strided_rows_and_errors(ops, oracle):
    rng = np.random.default_rng(2)
    big = torch.from_numpy(rng.standard_normal((5, 512)).astype(np.float16)).cuda()
    view = big[:, :256]
    want = oracle.had_r_128(view.cpu().numpy().astype(np.float32)).astype(np.float16)
    got = ops.had_r_128(view).cpu().numpy()
    assert np.abs(got.astype(np.float32) - want.astype(np.float32)).max() < 2e-3
    with pytest.raises(ValueError):
        ops.had_r_128(big[:, :100])
    with pytest.raises(ValueError):
        ops.had_r_128(big[0])
