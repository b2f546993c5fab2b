"""The routed blocks around the stacked experts (ponyexl3_b200.moe), on the CPU with a stand-in
for the expert switch: softmax -> top-k -> renormalise, the shared-expert slot appended as the
last expert with a sigmoid gate (ponyexl3/mlx/exl3_moe.py:790-839), and Gemma4's router — RMS
norm, projection, top-k of raw scores, softmax over the selected, per-expert scale (:842-923)."""

from __future__ import annotations

import numpy as np
import pytest

torch = pytest.importorskip("torch")


class _Switch(torch.nn.Module):
    """Expert e maps x to (e + 1) * x: the weighted sum then shows which experts were used."""

    def __init__(self, num_experts):
        super().__init__()
        self.num_experts = num_experts

    def forward(self, x, indices):
        return (indices[..., None].float() + 1.0) * x[..., None, :].float()


def test_shared_expert_slot_is_one_more_routing_weight():
    from ponyexl3_b200.moe import EXL3MoEBlock

    rng = np.random.default_rng(0)
    E, D, T, k = 9, 16, 5, 2                      # 8 routed experts + the shared one stacked last
    gate = torch.from_numpy(rng.standard_normal((E - 1, D)).astype(np.float32))
    sg = torch.from_numpy(rng.standard_normal((1, D)).astype(np.float32))
    x = torch.from_numpy(rng.standard_normal((T, D)).astype(np.float32))
    blk = EXL3MoEBlock(gate, _Switch(E), k, norm_topk_prob=True, shared_gate_weight=sg)
    inds, scores = blk.route(x.reshape(1, T, D))
    assert inds.shape == (1, T, k + 1) and bool((inds[..., -1] == E - 1).all())
    g = np.exp(x.numpy() @ gate.numpy().T)
    g /= g.sum(-1, keepdims=True)
    top = np.sort(np.argsort(-g, axis=-1)[:, :k], axis=-1)
    assert (np.sort(inds[0, :, :k].numpy(), axis=-1) == top).all()
    want_shared = 1.0 / (1.0 + np.exp(-(x.numpy() @ sg.numpy().T)))
    assert np.allclose(scores[0, :, -1:].numpy(), want_shared, atol=1e-6)
    assert np.allclose(scores[0, :, :k].sum(-1).numpy(), 1.0, atol=1e-6)
    y = blk(x)
    want = np.zeros((T, D), dtype=np.float64)
    for t in range(T):
        for j in range(k + 1):
            want[t] += float(scores[0, t, j]) * (int(inds[0, t, j]) + 1) * x[t].numpy()
    assert np.allclose(y.float().numpy(), want, rtol=2e-3, atol=2e-3)


def test_gemma4_router_and_weighted_sum():
    from ponyexl3_b200.moe import EXL3Gemma4MoEBlock

    rng = np.random.default_rng(1)
    E, D, T, k, eps = 8, 32, 6, 3, 1e-6
    proj = torch.from_numpy(rng.standard_normal((E, D)).astype(np.float32))
    scale = torch.from_numpy(rng.uniform(0.5, 1.5, D).astype(np.float32))
    pes = torch.from_numpy(rng.uniform(0.5, 2.0, E).astype(np.float32))
    x = torch.from_numpy(rng.standard_normal((T, D)).astype(np.float32))
    blk = EXL3Gemma4MoEBlock(proj, scale, pes, _Switch(E), k, eps, hidden_size=D)
    inds, weights = blk(x)
    xn = x.numpy().astype(np.float64)
    normed = xn / np.sqrt((xn ** 2).mean(-1, keepdims=True) + eps) * (scale.numpy() * D ** -0.5)
    s = normed @ proj.numpy().T.astype(np.float64)
    for t in range(T):
        top = np.argsort(-s[t])[:k]
        assert sorted(inds[t].tolist()) == sorted(top.tolist())
        sel = s[t, inds[t].numpy()]
        w = np.exp(sel - sel.max())
        w = w / w.sum() * pes.numpy()[inds[t].numpy()]
        assert np.allclose(weights[t].numpy(), w, rtol=1e-4, atol=1e-6)
    y = blk(x, inds, weights)
    want = ((weights.numpy() * (inds.numpy() + 1.0)).sum(-1, keepdims=True)) * x.numpy()
    assert np.allclose(y.float().numpy(), want, rtol=2e-3, atol=2e-3)
