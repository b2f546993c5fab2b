"""GPU parity of the block-table GEMV users: fused sibling groups and the stacked-expert
SwitchGLU (decode and prefill paths), against the CPU oracle.  Tolerance 1e-3 relative L2 per
linear; the MoE chain (gate/up -> GLU -> down) is checked at 2e-3, as two roundings chain."""

from __future__ import annotations

import numpy as np
import pytest

from conftest import rel_err, synthetic_layer

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda")


def _members(k, inf, outs, seed, cb=0):
    import ponyexl3_b200
    layers = []
    for i, o in enumerate(outs):
        tr, suh, svh, _ = synthetic_layer(k, inf, o, seed + i)
        layers.append(ponyexl3_b200.EXL3Layer(f"m{i}", inf, o, k, tr, suh, svh, None,
                                              mcg=(cb == 1), mul1=(cb == 2)))
    return layers


@pytest.mark.parametrize("rows", [1, 8, 16, 19])
@pytest.mark.parametrize("k,cb", [(4, 0), (3, 1), (6, 2)])
def test_fused_group_matches_members(cuda, oracle, rows, k, cb):
    """Rows {1, 8, 19} as the reference's group test (tests/test_exl3_fused.py:31-45)."""
    from ponyexl3_b200.fused import FusedEXL3Group

    layers = _members(k, 512, [512, 128, 256], seed=900 + k, cb=cb)
    grp = FusedEXL3Group(layers)
    x = np.random.default_rng(rows).standard_normal((rows, 512)).astype(np.float16)
    outs = grp.forward_all(torch.from_numpy(x).cuda())
    assert len(outs) == 3
    for o, l in zip(outs, layers):
        want = oracle.linear_forward(x, l.trellis, l.k, l.codebook_mode, l.suh, l.svh, None)
        assert o.shape == want.shape
        assert rel_err(o.cpu().numpy(), want) <= 1e-3


def test_fused_siblings_share_one_launch_and_refuse_bad_groups(cuda):
    from ponyexl3_b200.fused import FusedEXL3Group, fusable

    layers = _members(4, 256, [256, 128], seed=950)
    grp = FusedEXL3Group(layers)
    q, kproj = grp.sibling(0), grp.sibling(1)
    x = torch.randn((1, 256), device="cuda").half()
    a = q(x)
    assert grp._cache_x is x
    b = kproj(x)
    assert a.shape == (1, 256) and b.shape == (1, 128)
    assert list(grp.parameters()) == []
    bad = _members(4, 256, [256, 128], seed=951)
    bad[1].k = 5
    assert not fusable(bad)
    with pytest.raises(ValueError):
        FusedEXL3Group(bad)


def _experts(E, D, H, k, seed):
    rng = np.random.default_rng(seed)
    gu = rng.integers(0, 65536, size=(D // 16, E * 2 * H // 16, 16 * k), dtype=np.uint16)
    dn = rng.integers(0, 65536, size=(H // 16, E * D // 16, 16 * k), dtype=np.uint16)
    sg = lambda *s: np.where(rng.random(s) > 0.5, -1.0, 1.0).astype(np.float16)
    return dict(gu_trellis=gu, gu_suh=sg(E, 2, D), gu_svh=sg(E, 2 * H), dn_trellis=dn,
                dn_suh=sg(E, H), dn_svh=sg(E, D))


def _switch(w, k, cb, act="silu"):
    from ponyexl3_b200.moe import EXL3SwitchGLU

    t = {n: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda() for n, a in w.items()}
    for n in ("gu_suh", "gu_svh", "dn_suh", "dn_svh"):
        t[n] = t[n].view(torch.float16)
    return EXL3SwitchGLU(**t, k=k, cb=cb, activation=act)


@pytest.mark.parametrize("tokens", [1, 3, 16])
@pytest.mark.parametrize("k,cb,act", [(4, 0, "silu"), (3, 1, "gelu")])
def test_switch_glu_decode_matches_oracle(cuda, oracle, tokens, k, cb, act):
    E, D, H, kk = 8, 256, 128, 2
    w = _experts(E, D, H, k, seed=40 + k)
    sw = _switch(w, k, cb, act)
    rng = np.random.default_rng(tokens)
    x = (rng.standard_normal((tokens, D)) * 0.5).astype(np.float16)
    idx = np.stack([rng.choice(E, size=kk, replace=False) for _ in range(tokens)]).astype(np.int64)
    y = sw(torch.from_numpy(x).cuda().view(1, tokens, D), torch.from_numpy(idx).cuda().view(1, tokens, kk))
    assert y.shape == (1, tokens, kk, D)
    want = oracle.switch_glu(x, idx, **w, k=k, cb=cb, activation=act)
    assert rel_err(y.cpu().numpy().reshape(tokens, kk, D), want) <= 2e-3


def test_switch_glu_prefill_matches_oracle_and_decode(cuda, oracle):
    E, D, H, kk, k = 8, 256, 128, 2, 4
    w = _experts(E, D, H, k, seed=77)
    sw = _switch(w, k, 0)
    rng = np.random.default_rng(5)
    T = 150
    x = (rng.standard_normal((T, D)) * 0.5).astype(np.float16)
    idx = np.stack([rng.choice(E, size=kk, replace=False) for _ in range(T)]).astype(np.int64)
    y = sw(torch.from_numpy(x).cuda().view(1, T, D), torch.from_numpy(idx).cuda().view(1, T, kk))
    want = oracle.switch_glu(x, idx, **w, k=k, cb=0)
    assert rel_err(y.cpu().numpy().reshape(T, kk, D), want) <= 2e-3


def test_config4_moe_block_one_token(cuda, oracle):
    """256 experts, top-8, hidden 2048, expert intermediate 512, K = 4: one token through router,
    stacked experts and weighted sum; expert outputs checked against the oracle."""
    from ponyexl3_b200.moe import EXL3MoEBlock, route_topk

    E, D, H, kk, k = 256, 2048, 512, 8, 4
    w = _experts(E, D, H, k, seed=4000)
    sw = _switch(w, k, 0)
    rng = np.random.default_rng(4001)
    # random trellis words decode to unit-variance weights: keep the chain inside fp16 range
    x = (rng.standard_normal((1, D)) * 0.02).astype(np.float16)
    logits = rng.standard_normal((1, E)).astype(np.float32)
    inds, scores = route_topk(torch.from_numpy(logits).cuda(), kk)
    assert abs(float(scores.sum()) - 1.0) < 1e-5
    y = sw(torch.from_numpy(x).cuda().view(1, 1, D), inds.view(1, 1, kk))
    want = oracle.switch_glu(x, inds.cpu().numpy(), **w, k=k, cb=0)
    assert rel_err(y.cpu().numpy().reshape(1, kk, D), want) <= 2e-3
    gate_w = torch.from_numpy(rng.standard_normal((E, D)).astype(np.float32) * 0.05).cuda()
    blk = EXL3MoEBlock(gate_w, sw, kk)
    out = blk(torch.from_numpy(x).cuda())
    assert out.shape == (1, D) and torch.isfinite(out.float()).all()


def test_config4_prefill_tile_table(cuda, oracle):
    """Config-4 expert dims with 128 tokens x top-8 = 1024 sorted pairs over 256 experts: most
    row tiles are ragged and many table slots stay unused."""
    E, D, H, kk, k = 256, 2048, 512, 8, 4
    w = _experts(E, D, H, k, seed=4100)
    sw = _switch(w, k, 0)
    rng = np.random.default_rng(4101)
    T = 128
    x = (rng.standard_normal((T, D)) * 0.02).astype(np.float16)
    idx = np.stack([rng.choice(E, size=kk, replace=False) for _ in range(T)]).astype(np.int64)
    y = sw(torch.from_numpy(x).cuda().view(1, T, D), torch.from_numpy(idx).cuda().view(1, T, kk))
    from ponyexl3_b200 import ops
    assert ops.Workspace.get(torch.device("cuda"), 1, 128).status() == 0
    want = oracle.switch_glu(x, idx, **w, k=k, cb=0)
    assert rel_err(y.cpu().numpy().reshape(T, kk, D), want) <= 2e-3


def test_config4_sixteen_tokens(cuda, oracle):
    """Config-4 dims with 16 tokens x top-8 = 128 (token, slot) pairs over about 100 distinct
    experts: the block-table GEMV with many blocks per CTA and a different sign vector per block."""
    from ponyexl3_b200 import ops
    from ponyexl3_b200.moe import route_topk

    E, D, H, kk, k, T = 256, 2048, 512, 8, 4, 16
    w = _experts(E, D, H, k, seed=4200)
    sw = _switch(w, k, 0)
    rng = np.random.default_rng(4201)
    x = (rng.standard_normal((T, D)) * 0.02).astype(np.float16)
    inds, _ = route_topk(torch.from_numpy(rng.standard_normal((1, T, E)).astype(np.float32)).cuda(), kk)
    y = sw(torch.from_numpy(x).cuda().view(1, T, D), inds.view(1, T, kk))
    assert ops.Workspace.get(torch.device("cuda"), 1, 128).status() == 0
    want = oracle.switch_glu(x, inds.reshape(T, kk).cpu().numpy(), **w, k=k, cb=0)
    assert rel_err(y.cpu().numpy().reshape(T, kk, D), want) <= 2e-3


def test_config4_4096_tokens_sampled(cuda, oracle):
    """Config-4 dims at 4096 tokens (32,768 pairs, full tile tables): every output row is finite
    and 256 sampled (token, slot) pairs match the oracle, each pair being independent of the rest."""
    from ponyexl3_b200 import ops
    from ponyexl3_b200.moe import route_topk

    E, D, H, kk, k, T = 256, 2048, 512, 8, 4, 4096
    w = _experts(E, D, H, k, seed=4300)
    sw = _switch(w, k, 0)
    rng = np.random.default_rng(4301)
    x = (rng.standard_normal((T, D)) * 0.02).astype(np.float16)
    inds, _ = route_topk(torch.from_numpy(rng.standard_normal((1, T, E)).astype(np.float32)).cuda(), kk)
    y = sw(torch.from_numpy(x).cuda().view(1, T, D), inds.view(1, T, kk))
    assert ops.Workspace.get(torch.device("cuda"), 1, 128).status() == 0
    y = y.cpu().numpy().reshape(T, kk, D)
    assert np.isfinite(y.astype(np.float32)).all()
    idx = inds.reshape(T, kk).cpu().numpy()
    toks = rng.choice(T, size=256, replace=False)
    slots = rng.integers(0, kk, size=256)
    want = oracle.switch_glu(x[toks], idx[toks, slots][:, None], **w, k=k, cb=0)[:, 0]
    assert rel_err(y[toks, slots], want) <= 2e-3


@pytest.mark.parametrize("world", [2, 3, 8])
@pytest.mark.parametrize("tokens", [1, 5, 16])
def test_decode_over_an_expert_range_sums_to_the_full_switch(cuda, oracle, world, tokens):
    """Expert parallelism for few tokens, every rank's share computed one after the other on this
    GPU: a rank holds a contiguous expert range, the library picks its pairs on the device (the
    count never reaches the host) and leaves the other pairs' rows zero; the shares add up to the
    oracle's output, and a captured replay gives the same values."""
    from ponyexl3_b200 import ops
    from ponyexl3_b200.parallel import shard_expert_weights, shard_experts

    E, D, H, kk, k = 16, 256, 128, 4, 4
    w = _experts(E, D, H, k, seed=910 + world)
    rng = np.random.default_rng(tokens * 10 + world)
    x = (rng.standard_normal((tokens, D)) * 0.5).astype(np.float16)
    idx = np.stack([rng.choice(E, size=kk, replace=False) for _ in range(tokens)]).astype(np.int64)
    xd, idd = torch.from_numpy(x).cuda(), torch.from_numpy(idx).cuda()
    total = torch.zeros((tokens, kk, D), dtype=torch.float32, device="cuda")
    nonzero_rows = 0
    for rank in range(world):
        e0, e1 = shard_experts(E, world, rank)
        sw = _switch(shard_expert_weights(w, E, world, rank), k, 0)
        y = sw.decode_range(xd, idd, (e0, e1, E))
        held = (idd >= e0) & (idd < e1)
        assert bool((y[~held] == 0).all())                      # nobody else's rows are touched
        nonzero_rows += int(held.sum())
        if rank == 0:                                           # the same call from a CUDA graph
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                sw.decode_range(xd, idd, (e0, e1, E))
                stream.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    yg = sw.decode_range(xd, idd, (e0, e1, E))
                graph.replay()
                stream.synchronize()
            assert torch.equal(yg, y)
        total += y.float()
    assert nonzero_rows == tokens * kk
    assert ops.Workspace.get(torch.device("cuda"), 1, 128).status() == 0
    want = oracle.switch_glu(x, idx, **w, k=k, cb=0)
    assert rel_err(total.cpu().numpy(), want) <= 2e-3


@pytest.mark.parametrize("world,act,T,kk", [(2, "silu", 96, 4), (4, "silu", 96, 4), (2, "gelu", 96, 4), (4, "gelu", 96, 4),
                                            (2, "silu", 20, 2)])
def test_prefill_over_an_expert_range_stores_rows_at_their_owners(cuda, oracle, world, act, T, kk):
    """Expert parallelism for many tokens, every rank's share computed one after the other on
    this GPU: tokens are partitioned (buffer p holds the output rows of partition p), a rank
    sorts and tiles only the pairs of its experts (their number stays on the device), its down
    projection stores each row into the owner's buffer and announces itself on every owner's
    counter.  After all ranks every counter holds `world` arrivals and the buffers hold the
    oracle's output."""
    import ctypes

    from ponyexl3_b200 import ops
    from ponyexl3_b200.parallel import shard_expert_weights, shard_experts

    E, D, H, k = 16, 256, 128, 4            # the last case: fewer than 64 pairs in all
    w = _experts(E, D, H, k, seed=930 + world)
    rng = np.random.default_rng(31 + world)
    x = (rng.standard_normal((T, D)) * 0.5).astype(np.float16)
    idx = np.stack([rng.choice(E, size=kk, replace=False) for _ in range(T)]).astype(np.int64)
    xd, idd = torch.from_numpy(x).cuda(), torch.from_numpy(idx).cuda()
    n_local = T // world * kk
    bufs = [torch.full((n_local, D), float("nan"), dtype=torch.float16, device="cuda") for _ in range(world)]
    ctrs = torch.zeros(world * 64, dtype=torch.int32, device="cuda")      # counters 256 bytes apart
    u64 = ctypes.c_uint64 * world
    y_ptrs = u64(*[b.data_ptr() for b in bufs])
    c_ptrs = u64(*[ctrs.data_ptr() + 256 * p for p in range(world)])
    for rank in range(world):
        e0, e1 = shard_experts(E, world, rank)
        sw = _switch(shard_expert_weights(w, E, world, rank), k, 0, act)
        sw.prefill_range(xd, idd, (e0, e1, E), (y_ptrs, c_ptrs, world, n_local, D))
    torch.cuda.synchronize()
    assert ctrs.view(world, 64)[:, 0].tolist() == [world] * world
    assert ops.Workspace.get(torch.device("cuda"), 1, 128).status() == 0
    got = torch.cat(bufs).cpu().numpy().reshape(T, kk, D)
    assert np.isfinite(got.astype(np.float32)).all()          # every row was written by somebody
    want = oracle.switch_glu(x, idx, **w, k=k, cb=0, activation=act)
    assert rel_err(got, want) <= 2e-3


@pytest.mark.parametrize("act", ["silu", "gelu"])
@pytest.mark.parametrize("rows", [1, 3, 8, 16])
def test_glu_folded_into_the_down_projection(cuda, oracle, act, rows):
    """EXL3_FLAG_GLU_*: the GEMV reads [gate | up] rows and applies the activation while loading —
    same result as the oracle's GLU (fp16 h) followed by its linear forward, for the fused
    rotation (few rows) and the rotation-kernel path (many rows)."""
    from ponyexl3_b200 import ops

    H, D, k, cb = 1024, 512, 4, 0
    tr, suh, svh, _ = synthetic_layer(k, H, D, seed=700 + rows)
    rng = np.random.default_rng(rows)
    gu = (rng.standard_normal((rows, 2 * H)) * 1.5).astype(np.float16)
    h = oracle.glu(gu[:, :H], gu[:, H:], act)
    want = oracle.linear_forward(h, tr, k, cb, suh, svh, None)
    t = lambda a: torch.from_numpy(a).cuda()
    y = ops.gemv(t(gu), t(tr.view(np.int16)), k, cb, t(suh), t(svh), None, glu=act)
    assert rel_err(y.cpu().numpy(), want) <= 1e-3
    assert ops.Workspace.get(torch.device("cuda"), 1, 128).status() == 0


@pytest.mark.parametrize("rows", [1, 5, 16, 40])
def test_mlp_monolith_matches_the_three_linears(cuda, oracle, rows):
    """gate|up -> SiLU-GLU -> down as one module (the reference's EXL3MLPMonolith): equals the
    oracle's chain of linear forwards with h rounded to fp16 in between."""
    import ponyexl3_b200
    from ponyexl3_b200.fused import FusedEXL3Group
    from ponyexl3_b200.linear import EXL3Linear
    from ponyexl3_b200.mlp import EXL3MLPMonolith

    D, H, k = 512, 1024, 4
    gate, up = _members(k, D, [H, H], seed=1300)
    trd, suhd, svhd, _ = synthetic_layer(k, H, D, seed=1310)
    down = ponyexl3_b200.EXL3Layer("down", H, D, k, trd, suhd, svhd, None)
    mlp = EXL3MLPMonolith.from_fused_gate_up(FusedEXL3Group([gate, up]), EXL3Linear(down))
    x = (np.random.default_rng(rows).standard_normal((rows, D)) * 0.05).astype(np.float16)
    y = mlp(torch.from_numpy(x).cuda())
    g = oracle.linear_forward(x, gate.trellis, k, 0, gate.suh, gate.svh, None)
    u = oracle.linear_forward(x, up.trellis, k, 0, up.suh, up.svh, None)
    want = oracle.linear_forward(oracle.glu(g, u, "silu"), trd, k, 0, suhd, svhd, None)
    assert y.shape == (rows, D)
    assert rel_err(y.cpu().numpy(), want) <= 2e-3
