"""The decode-step kernels around the EXL3 linears (residual + RMSNorm, rotary + cache append,
grouped-query decode attention, SwiGLU) against plain PyTorch fp32 restatements of the same math."""

import math

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from ponyexl3_b200 import ops as o
    return o


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm())


@pytest.mark.parametrize("rows,n,with_delta", [(1, 5120, True), (16, 5120, True), (3, 256, False), (2, 17408, True)])
def test_add_rmsnorm(ops, rows, n, with_delta):
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn((rows, n), device="cuda", generator=g).half()
    d = torch.randn((rows, n), device="cuda", generator=g).half() if with_delta else None
    w = (1 + 0.1 * torch.randn(n, device="cuda", generator=g)).half()
    want_x = (x + d) if with_delta else x.clone()          # fp16 add, as the residual stream does
    xf = want_x.float()
    want_h = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + 1e-6) * w.float()
    h = ops.add_rmsnorm(x, d, w, 1e-6)
    assert torch.equal(x, want_x)
    assert _rel(h, want_h) < 1e-3


@pytest.mark.parametrize("rows,hq,hkv", [(1, 40, 8), (16, 40, 8), (3, 5, 1)])
def test_rope_append(ops, rows, hq, hkv):
    g = torch.Generator(device="cuda").manual_seed(2)
    cache_len, pos0 = 64, 40
    qkv = torch.randn((rows, (hq + 2 * hkv) * 128), device="cuda", generator=g).half()
    ang = torch.rand((rows, 64), device="cuda", generator=g) * 6.28
    cos = torch.cat([ang.cos(), ang.cos()], -1).half()
    sin = torch.cat([ang.sin(), ang.sin()], -1).half()
    kc = torch.randn((hkv, cache_len, 128), device="cuda", generator=g).half()
    vc = torch.randn((hkv, cache_len, 128), device="cuda", generator=g).half()
    kc0, vc0 = kc.clone(), vc.clone()
    q = ops.rope_append(qkv, cos, sin, kc, vc, hq, pos0)

    def rope(t):                                               # (rows, heads, 128) fp32
        rot = torch.cat([-t[..., 64:], t[..., :64]], -1)
        return t * cos.float()[:, None] + rot * sin.float()[:, None]

    t = qkv.float().view(rows, hq + 2 * hkv, 128)
    assert _rel(q, rope(t[:, :hq])) < 1e-3
    assert _rel(kc[:, pos0:pos0 + rows], rope(t[:, hq:hq + hkv]).transpose(0, 1)) < 1e-3
    assert torch.equal(vc[:, pos0:pos0 + rows], qkv.view(rows, -1, 128)[:, hq + hkv:].transpose(0, 1))
    keep = torch.ones(cache_len, dtype=torch.bool, device="cuda")
    keep[pos0:pos0 + rows] = False
    assert torch.equal(kc[:, keep], kc0[:, keep]) and torch.equal(vc[:, keep], vc0[:, keep])


@pytest.mark.parametrize("rows,h", [(1, 17408), (16, 17408), (2, 2176), (5, 512)])
def test_swiglu(ops, rows, h):
    g = torch.Generator(device="cuda").manual_seed(3)
    gu = torch.randn((rows, 2 * h), device="cuda", generator=g).half()
    want = torch.nn.functional.silu(gu[:, :h].float()) * gu[:, h:].float()
    assert _rel(ops.swiglu(gu), want) < 1e-3


def _attention_reference(q, kc, vc, ctx):
    rows, hq, _ = q.shape
    hkv = kc.shape[0]
    group = hq // hkv
    total = ctx + rows
    k = kc[:, :total].float().repeat_interleave(group, dim=0)      # (hq, total, 128)
    v = vc[:, :total].float().repeat_interleave(group, dim=0)
    s = torch.einsum("rhd,htd->hrt", q.float(), k) / math.sqrt(128)
    pos = torch.arange(total, device=q.device)
    mask = pos[None, :] <= (ctx + torch.arange(rows, device=q.device))[:, None]
    s = s.masked_fill(~mask[None], float("-inf"))
    return torch.einsum("hrt,htd->rhd", torch.softmax(s, -1), v).reshape(rows, hq * 128)


@pytest.mark.parametrize("rows,hq,hkv,ctx", [
    (1, 40, 8, 8192), (16, 40, 8, 8192),        # the 27B-class decode and verify shapes
    (1, 5, 1, 8192), (16, 5, 1, 8192),          # one KV head per rank (8-way tensor parallel)
    (3, 8, 2, 100), (1, 5, 1, 63), (1, 5, 1, 0), (7, 16, 2, 129), (16, 8, 1, 500), (2, 4, 4, 4097)])
def test_attn_decode(ops, rows, hq, hkv, ctx):
    g = torch.Generator(device="cuda").manual_seed(4)
    cache_len = ctx + 16
    q = torch.randn((rows, hq, 128), device="cuda", generator=g).half()
    kc = torch.randn((hkv, cache_len, 128), device="cuda", generator=g).half()
    vc = torch.randn((hkv, cache_len, 128), device="cuda", generator=g).half()
    out = ops.attn_decode(q, kc, vc, ctx)
    want = _attention_reference(q, kc, vc, ctx)
    assert out.shape == (rows, hq * 128)
    assert torch.isfinite(out.float()).all()
    assert _rel(out, want) < 2e-3


def test_attn_decode_peaked_scores(ops):
    """Large logits: the running-maximum bookkeeping across tiles and chunks must hold."""
    g = torch.Generator(device="cuda").manual_seed(5)
    rows, hq, hkv, ctx = 4, 10, 2, 3000
    q = (torch.randn((rows, hq, 128), device="cuda", generator=g) * 4).half()
    kc = (torch.randn((hkv, ctx + 16, 128), device="cuda", generator=g) * 4).half()
    vc = torch.randn((hkv, ctx + 16, 128), device="cuda", generator=g).half()
    assert _rel(ops.attn_decode(q, kc, vc, ctx), _attention_reference(q, kc, vc, ctx)) < 3e-3


@pytest.mark.parametrize("rows", [1, 4])
def test_dense_step_native_glue_matches_torch_glue(rows):
    from ponyexl3_b200.dense_step import DenseConfig, SyntheticDenseDecoder
    from torch_glue_decoder import TorchGlueDecoder
    cfg = DenseConfig(layers=2, hidden=512, intermediate=768, q_heads=4, kv_heads=2, head_dim=128,
                      vocab=1152, context=200, max_rows=4)
    dev = torch.device("cuda", 0)
    a = SyntheticDenseDecoder(cfg, dev, seed=31)
    b = TorchGlueDecoder(cfg, dev, seed=31)
    tok = torch.tensor([9, 800, 77, 1000][:rows], device=dev)
    la, lb = a.forward_logits(tok), b.forward_logits(tok)
    assert _rel(la, lb) < 1e-2
    # the caches were appended identically (within the rotary rounding)
    for La, Lb in zip(a.layers, b.layers):
        assert _rel(La.k_cache[:, :cfg.context + rows], Lb.k_cache[:, :cfg.context + rows]) < 2e-3
        assert _rel(La.v_cache[:, :cfg.context + rows], Lb.v_cache[:, :cfg.context + rows]) < 2e-3
