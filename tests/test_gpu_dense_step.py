"""The decode step around the EXL3 path (dense_step.SyntheticDenseDecoder) against a CPU
restatement that runs every linear through the oracle and the glue in fp32."""

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _np16(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.float16)


def _npu16(t):
    return t.detach().cpu().contiguous().numpy().view(np.uint16)


def _lin(oracle, x, m):
    return oracle.linear_forward(x.astype(np.float16), _npu16(m._trellis), m.k, m.cb, _np16(m._suh),
                                 _np16(m._svh), None).astype(np.float32)


def _group(oracle, x, g):
    outs, tr = [], _npu16(g._trellis)
    suh, svh = _np16(g._suh_stack), _np16(g._svh_cat)
    for i, n in enumerate(g._out_features):
        a = int(g._offsets[i])
        outs.append(oracle.linear_forward(x.astype(np.float16), np.ascontiguousarray(tr[:, a // 16:(a + n) // 16]),
                                          g.k, g.cb, suh[i], svh[a:a + n], None).astype(np.float32))
    return outs


def _rms(x, eps):
    x = x.astype(np.float32)
    return (x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)).astype(np.float16)


def _rope(t, cos, sin):
    half = t.shape[-1] // 2
    rot = np.concatenate([-t[..., half:], t[..., :half]], axis=-1)
    return t * cos[:, None, :] + rot * sin[:, None, :]


def _reference_logits(oracle, dec, tokens, k_caches, v_caches):
    c = dec.cfg
    rows, hd = len(tokens), c.head_dim
    cos, sin = _np16(dec.cos).astype(np.float32)[:rows], _np16(dec.sin).astype(np.float32)[:rows]
    x = _np16(dec.embed)[tokens].astype(np.float32)
    for li, L in enumerate(dec.layers):
        h = _rms(x, c.rms_eps)
        q, k, v = _group(oracle, h, L.qkv)
        q = _rope(q.reshape(rows, c.q_heads, hd), cos, sin)
        k = _rope(k.reshape(rows, c.kv_heads, hd), cos, sin)
        v = v.reshape(rows, c.kv_heads, hd)
        kc = np.concatenate([k_caches[li][:, :c.context].astype(np.float32), k.transpose(1, 0, 2)], axis=1)
        vc = np.concatenate([v_caches[li][:, :c.context].astype(np.float32), v.transpose(1, 0, 2)], axis=1)
        out = np.zeros((rows, c.q_heads, hd), dtype=np.float32)
        for r in range(rows):
            n = c.context + r + 1
            for hq in range(c.q_heads):
                kv = hq // c.group
                s = kc[kv, :n] @ q[r, hq] / np.sqrt(hd)
                p = np.exp(s - s.max())
                out[r, hq] = (p / p.sum()) @ vc[kv, :n]
        x = (x + _lin(oracle, out.reshape(rows, -1), L.o)).astype(np.float16).astype(np.float32)
        h = _rms(x, c.rms_eps)
        g, u = _group(oracle, h, L.gate_up)
        act = (g / (1.0 + np.exp(-g))) * u
        x = (x + _lin(oracle, act, L.down)).astype(np.float16).astype(np.float32)
    return _lin(oracle, _rms(x, c.rms_eps), dec.head)


@pytest.mark.parametrize("rows", [1, 4])
def test_decode_step_matches_cpu_restatement(oracle, rows):
    from ponyexl3_b200.dense_step import DenseConfig, SyntheticDenseDecoder
    cfg = DenseConfig(layers=2, hidden=512, intermediate=512, q_heads=4, kv_heads=2, head_dim=128,
                      vocab=1024, context=48, max_rows=4, k5_fraction=0.5)
    dev = torch.device("cuda", 0)
    dec = SyntheticDenseDecoder(cfg, dev, seed=11)
    assert set(dec.ks) <= {4, 5}
    k_caches = [_np16(L.k_cache) for L in dec.layers]       # before the step writes new positions
    v_caches = [_np16(L.v_cache) for L in dec.layers]
    tokens = torch.tensor([5, 900, 17, 333][:rows], device=dev)
    logits = dec.forward_logits(tokens).float().cpu().numpy()
    ref = _reference_logits(oracle, dec, tokens.cpu().numpy(), k_caches, v_caches)
    err = np.linalg.norm(logits - ref) / np.linalg.norm(ref)
    assert err < 2e-2, err
    nxt = dec.step(tokens).cpu().numpy()
    # arg-max agrees wherever the reference's top-2 margin exceeds the error scale
    top2 = np.sort(ref, axis=-1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 0.05 * np.abs(ref).max()
    assert np.array_equal(nxt[clear], ref.argmax(-1)[clear])


def test_step_is_graph_capturable_and_deterministic():
    from ponyexl3_b200.dense_step import DenseConfig, SyntheticDenseDecoder
    cfg = DenseConfig(layers=2, hidden=512, intermediate=512, q_heads=4, kv_heads=2, head_dim=128,
                      vocab=1024, context=48, max_rows=4)
    dev = torch.device("cuda", 0)
    dec = SyntheticDenseDecoder(cfg, dev, seed=12)
    tokens = torch.tensor([7], device=dev)
    eager = dec.step(tokens).clone()
    s = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(s):
        dec.step(tokens)
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            out = dec.step(tokens)
        g.replay()
        g.replay()
        s.synchronize()
    assert torch.equal(out, eager)
