"""GPU parity of the linear forward (rows 1..16) through the module and the C ABI,
against the CPU oracle and the golden forwards made by the reference.
Tolerance: relative L2 error <= 1e-3 (fp32 accumulate), as the target states."""

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
    layer = mod.EXL3Layer("test", inf, outf, k, tr, suh, svh, b, mcg=(cb == 1), mul1=(cb == 2))
    return layer


def _check(mod, oracle, layer, x, tol=REL_TOL):
    m = mod.EXL3Linear(layer)
    y = m(torch.from_numpy(x).cuda()).cpu().numpy()
    want = oracle.linear_forward(x, layer.trellis, layer.k, layer.codebook_mode, layer.suh,
                                 layer.svh, layer.bias)
    assert y.shape == want.shape and y.dtype == np.float16
    assert np.isfinite(y.astype(np.float32)).all()
    e = rel_err(y, want)
    assert e <= tol, f"rel err {e}"
    assert mod.ops.Workspace.get(torch.device("cuda"), 1, 128).status() == 0
    return y, want


def test_golden_forwards_from_the_reference(mod, golden):
    g = golden["forward"]
    for i in range(int(g["n_cases"][0])):
        k, mcg, mul1, inf, outf, rows, has_bias = (int(v) for v in g[f"c{i}_meta"])
        layer = mod.EXL3Layer(f"c{i}", inf, outf, k, g[f"c{i}_trellis"],
                              g[f"c{i}_suh"].view(np.float16), g[f"c{i}_svh"].view(np.float16),
                              g[f"c{i}_bias"].view(np.float16) if has_bias else None,
                              mcg=bool(mcg), mul1=bool(mul1))
        x = g[f"c{i}_x"].view(np.float16)
        y = mod.EXL3Linear(layer)(torch.from_numpy(x).cuda()).cpu().numpy()
        assert rel_err(y, g[f"c{i}_y"].view(np.float16)) <= REL_TOL, f"case {i}"
    layer = mod.EXL3Layer("ps", 128, 128, 3, g["packed_signs_trellis"], g["packed_signs_su"],
                          g["packed_signs_sv"])
    y = mod.EXL3Linear(layer)(torch.from_numpy(g["packed_signs_x"].view(np.float16)).cuda())
    assert rel_err(y.cpu().numpy(), g["packed_signs_y"].view(np.float16)) <= REL_TOL


@pytest.mark.parametrize("k", range(1, 9))
@pytest.mark.parametrize("cb", [0, 1, 2])
def test_gemv_all_k_all_codebooks(mod, oracle, k, cb):
    layer = _layer(mod, k, 512, 384, seed=50 + 10 * k + cb, cb=cb, bias=(k % 2 == 0))
    rng = np.random.default_rng(k)
    for rows in (1, 5, 16):
        x = rng.standard_normal((rows, 512)).astype(np.float16)
        _check(mod, oracle, layer, x)


@pytest.mark.parametrize("rows", [1, 2, 3, 4, 7, 8, 9, 12, 16])
def test_gemv_row_counts(mod, oracle, rows):
    layer = _layer(mod, 4, 1024, 640, seed=7)
    x = np.random.default_rng(rows).standard_normal((rows, 1024)).astype(np.float16)
    _check(mod, oracle, layer, x)


def test_config1_single_layer(mod, oracle):
    """in = out = 4096, K = 4, 3INST, x [1, 4096] fp16 N(0,1)."""
    layer = _layer(mod, 4, 4096, 4096, seed=1000)
    x = np.random.default_rng(1001).standard_normal((1, 4096)).astype(np.float16)
    _check(mod, oracle, layer, x)


@pytest.mark.parametrize("shape", [(5120, 17408), (17408, 5120), (5120, 5120)])
@pytest.mark.parametrize("rows", [1, 16])
def test_config2_shapes_k4(mod, oracle, shape, rows):
    """Full benchmark shapes: many CTAs share each column block (split-K fix-up)."""
    layer = _layer(mod, 4, shape[0], shape[1], seed=2000 + rows)
    x = np.random.default_rng(rows).standard_normal((rows, shape[0])).astype(np.float16)
    _check(mod, oracle, layer, x)


FULL_SHAPES = [(5120, 17408), (17408, 5120), (5120, 5120)]


@pytest.mark.parametrize("k,cb", [(k, cb) for k in (1, 3, 5, 8) for cb in (1, 2)] +
                         [(2, 0), (5, 0), (6, 0), (7, 0)])
def test_config2_full_shapes_other_k_and_codebooks(mod, oracle, k, cb):
    """The sweep configuration at its real sizes away from K=4 / 3INST: one of the three
    shapes per (K, codebook), rows 1, 8 and 16 (fused rotation, one and two MMA row groups)."""
    inf, outf = FULL_SHAPES[(k + cb) % 3] if (k, cb) != (5, 0) else (17408, 5120)
    layer = _layer(mod, k, inf, outf, seed=2100 + 10 * k + cb, cb=cb)
    m = mod.EXL3Linear(layer)
    for rows in (1, 8, 16):
        x = np.random.default_rng(100 * k + rows).standard_normal((rows, inf)).astype(np.float16)
        y = m(torch.from_numpy(x).cuda()).cpu().numpy()
        want = oracle.linear_forward(x, layer.trellis, k, cb, layer.suh, layer.svh, None)
        e = rel_err(y, want)
        assert e <= REL_TOL, f"K={k} cb={cb} rows={rows} {inf}x{outf}: rel err {e}"
    assert mod.ops.Workspace.get(torch.device("cuda"), 1, 128).status() == 0


def test_fast_accum_on_the_golden_forwards(mod, golden):
    """EXL3_FLAG_FAST_ACCUM against the forwards the reference itself produced (3INST / MCG
    cases; MUL1 has no two-halves form and ignores the flag)."""
    g = golden["forward"]
    worst = 0.0
    for i in range(int(g["n_cases"][0])):
        k, mcg, mul1, inf, outf, rows, has_bias = (int(v) for v in g[f"c{i}_meta"])
        layer = mod.EXL3Layer(f"c{i}", inf, outf, k, g[f"c{i}_trellis"],
                              g[f"c{i}_suh"].view(np.float16), g[f"c{i}_svh"].view(np.float16),
                              g[f"c{i}_bias"].view(np.float16) if has_bias else None,
                              mcg=bool(mcg), mul1=bool(mul1))
        m = mod.EXL3Linear(layer)
        m.fast_accum = True
        y = m(torch.from_numpy(g[f"c{i}_x"].view(np.float16)).cuda()).cpu().numpy()
        e = rel_err(y, g[f"c{i}_y"].view(np.float16))
        worst = max(worst, e)
        assert e <= REL_TOL, f"case {i}: rel err {e}"
    assert worst > 0.0          # the mode really is a different rounding


@pytest.mark.parametrize("shape", [(4096, 4096)] + FULL_SHAPES)
@pytest.mark.parametrize("rows", [1, 16])
def test_fast_accum_full_shapes(mod, oracle, shape, rows):
    """The single-layer and sweep shapes at K=4 / 3INST in fast-accumulate mode."""
    layer = _layer(mod, 4, shape[0], shape[1], seed=2300 + rows)
    m = mod.EXL3Linear(layer)
    m.fast_accum = True
    x = np.random.default_rng(rows).standard_normal((rows, shape[0])).astype(np.float16)
    y = m(torch.from_numpy(x).cuda()).cpu().numpy()
    want = oracle.linear_forward(x, layer.trellis, 4, 0, layer.suh, layer.svh, None)
    assert rel_err(y, want) <= REL_TOL


def test_repeated_calls_are_deterministic_and_counters_rearm(mod, oracle):
    layer = _layer(mod, 5, 2048, 1024, seed=3)
    m = mod.EXL3Linear(layer)
    x = torch.from_numpy(np.random.default_rng(0).standard_normal((3, 2048)).astype(np.float16)).cuda()
    ys = [m(x).clone() for _ in range(5)]
    for y in ys[1:]:
        assert torch.equal(y, ys[0])


def test_linearity_in_x_at_full_size(mod):
    """Size-independent property: f(a) + f(b) ~= f(a + b) for the bias-free layer."""
    layer = _layer(mod, 4, 5120, 5120, seed=11)
    m = mod.EXL3Linear(layer)
    rng = np.random.default_rng(5)
    a = torch.from_numpy(rng.standard_normal((1, 5120)).astype(np.float16)).cuda()
    b = torch.from_numpy(rng.standard_normal((1, 5120)).astype(np.float16)).cuda()
    lhs = m(a).float() + m(b).float()
    rhs = m((a.float() + b.float()).half()).float()
    assert (lhs - rhs).norm() / rhs.norm() < 3e-3


def test_dtypes_shapes_and_no_parameters(mod, oracle):
    layer = _layer(mod, 4, 256, 384, seed=9, bias=True)
    m = mod.EXL3Linear(layer)
    assert list(m.parameters()) == [] and list(m.buffers()) == []
    x = np.random.default_rng(1).standard_normal((2, 3, 256)).astype(np.float32)
    y = m(torch.from_numpy(x).cuda())
    assert y.shape == (2, 3, 384) and y.dtype == torch.float16
    want = oracle.linear_forward(x.astype(np.float16), layer.trellis, 4, 0, layer.suh, layer.svh, layer.bias)
    assert rel_err(y.cpu().numpy(), want) <= REL_TOL
    xb = torch.from_numpy(x).cuda().to(torch.bfloat16)
    yb = m(xb)
    wantb = oracle.linear_forward(xb.float().cpu().numpy().astype(np.float16), layer.trellis, 4, 0,
                                  layer.suh, layer.svh, layer.bias)
    assert rel_err(yb.cpu().numpy(), wantb) <= REL_TOL
    assert m(torch.zeros((0, 256), device="cuda", dtype=torch.float16)).shape == (0, 384)
    with pytest.raises(ValueError):
        m(torch.zeros((1, 128), device="cuda", dtype=torch.float16))
    # no sign vectors at all
    layer2 = mod.EXL3Layer("nosign", 256, 384, 4, layer.trellis)
    x1 = x.reshape(-1, 256)[:1].astype(np.float16)
    y2 = mod.EXL3Linear(layer2)(torch.from_numpy(x1).cuda()).cpu().numpy()
    assert rel_err(y2, oracle.linear_forward(x1, layer.trellis, 4, 0, None, None)) <= REL_TOL


@pytest.mark.parametrize("k", [2, 4, 5, 8])
@pytest.mark.parametrize("cb", [0, 1, 2])
@pytest.mark.parametrize("rows", [1, 11])
def test_fast_accum_mode_stays_within_tolerance(mod, oracle, k, cb, rows):
    """EXL3_FLAG_FAST_ACCUM adds the two fp16 halves of a codebook value inside the fp32
    accumulation instead of rounding their sum first: same 1e-3 bound."""
    layer = _layer(mod, k, 2048, 512, seed=300 + k + cb, cb=cb)
    m = mod.EXL3Linear(layer)
    m.fast_accum = True
    x = np.random.default_rng(rows).standard_normal((rows, 2048)).astype(np.float16)
    y = m(torch.from_numpy(x).cuda()).cpu().numpy()
    want = oracle.linear_forward(x, layer.trellis, k, cb, layer.suh, layer.svh, None)
    assert rel_err(y, want) <= REL_TOL


def test_more_than_16_rows_go_to_the_gemm(mod, oracle):
    layer = _layer(mod, 3, 384, 256, seed=4)
    x = np.random.default_rng(2).standard_normal((37, 384)).astype(np.float16)
    _check(mod, oracle, layer, x)


def test_programmatic_launch_chain(mod, oracle):
    """Back-to-back layers launched with programmatic stream serialisation give the same
    results as plain launches."""
    layers = [_layer(mod, 4, 1024, 1024, seed=60 + i) for i in range(4)]
    mods = [mod.EXL3Linear(l) for l in layers]
    x = torch.from_numpy(np.random.default_rng(3).standard_normal((1, 1024)).astype(np.float16)).cuda()

    def chain(pdl):
        h = x
        for m in mods:
            m.pdl = pdl
            h = (m(h).float() * 0.05).half()
        return h

    plain = chain(False)
    for _ in range(3):
        assert torch.equal(chain(True), plain)
