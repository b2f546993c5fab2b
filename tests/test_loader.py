"""Checkpoint directory -> EXL3Layer (host only).  Behaviour follows ponyexl3/ref/loader.py:84-173
and the multiplier check of ponyexl3/mlx/model.py:261-283."""

import json

import numpy as np
import pytest

from ponyexl3_b200.layer import EXL3Layer
from ponyexl3_b200.loader import (CheckpointError, EXL3Checkpoint, has_exl3_layer_weights,
                                  list_exl3_layers, load_exl3_layer, save_exl3_layers)


def _layer(key, k, n_in, n_out, seed, bias=False, mcg=False, mul1=False, packed_signs=False):
    rng = np.random.default_rng(seed)
    trellis = rng.integers(0, 65536, size=(n_in // 16, n_out // 16, 16 * k), dtype=np.uint16)
    if packed_signs:
        suh = rng.integers(-32768, 32767, size=n_in // 16, dtype=np.int16)
        svh = rng.integers(-32768, 32767, size=n_out // 16, dtype=np.int16)
    else:
        suh = rng.choice([-1.0, 1.0], n_in).astype(np.float16)
        svh = (rng.choice([-1.0, 1.0], n_out) * rng.uniform(0.5, 2, n_out)).astype(np.float16)
    return EXL3Layer(key=key, in_features=n_in, out_features=n_out, k=k, trellis=trellis, suh=suh,
                     svh=svh, bias=rng.standard_normal(n_out).astype(np.float16) if bias else None,
                     mcg=mcg, mul1=mul1)


def _same(a: EXL3Layer, b: EXL3Layer):
    assert (a.key, a.in_features, a.out_features, a.k, a.mcg, a.mul1) == \
           (b.key, b.in_features, b.out_features, b.k, b.mcg, b.mul1)
    assert b.trellis.dtype == np.uint16 and np.array_equal(a.trellis, b.trellis)
    for name in ("suh", "svh", "bias"):
        x, y = getattr(a, name), getattr(b, name)
        assert (x is None) == (y is None)
        if x is not None:
            assert x.dtype == y.dtype and np.array_equal(x, y)


LAYERS = [
    _layer("model.layers.0.mlp.gate_proj", 4, 256, 384, 1),
    _layer("model.layers.0.mlp.down_proj", 3, 384, 256, 2, bias=True, mcg=True),
    _layer("model.layers.0.self_attn.q_proj", 8, 128, 128, 3, mul1=True),
    _layer("model.layers.1.self_attn.o_proj", 1, 128, 256, 4, packed_signs=True),
]


@pytest.mark.parametrize("shards", [1, 3])
def test_round_trip(tmp_path, shards):
    save_exl3_layers(tmp_path, LAYERS, shards=shards)
    assert (tmp_path / "model.safetensors.index.json").is_file() == (shards > 1)
    assert list_exl3_layers(tmp_path) == sorted(l.key for l in LAYERS)
    ck = EXL3Checkpoint(tmp_path)
    for l in LAYERS:
        assert has_exl3_layer_weights(tmp_path, l.key)
        _same(l, load_exl3_layer(tmp_path, l.key))
        _same(l, ck.layer(l.key))
    assert [l.key for l in ck.layers()] == ck.keys()


def test_k_and_shape_follow_the_trellis(tmp_path):
    save_exl3_layers(tmp_path, LAYERS)
    for l in LAYERS:
        got = load_exl3_layer(tmp_path, l.key)
        assert got.k == l.trellis.shape[2] // 16
        assert (got.in_features, got.out_features) == (l.trellis.shape[0] * 16, l.trellis.shape[1] * 16)


def test_non_exl3_records_and_missing_tensors_are_not_layers(tmp_path):
    save_exl3_layers(tmp_path, LAYERS[:1])
    cfg_path = tmp_path / "quantization_config.json"
    cfg = json.loads(cfg_path.read_text())
    cfg["tensor_storage"]["model.embed_tokens"] = {"quant_format": "fp16"}
    cfg["tensor_storage"]["model.layers.9.mlp.up_proj"] = {"quant_format": "exl3"}   # no tensors
    cfg_path.write_text(json.dumps(cfg))
    assert list_exl3_layers(tmp_path) == [LAYERS[0].key]
    assert not has_exl3_layer_weights(tmp_path, "model.embed_tokens")
    assert not has_exl3_layer_weights(tmp_path, "model.layers.9.mlp.up_proj")
    with pytest.raises(CheckpointError):
        load_exl3_layer(tmp_path, "model.embed_tokens")
    with pytest.raises(CheckpointError):
        load_exl3_layer(tmp_path, "model.layers.9.mlp.up_proj")


def test_missing_config(tmp_path):
    with pytest.raises(CheckpointError):
        list_exl3_layers(tmp_path)


@pytest.mark.parametrize("name,flag", [("mcg", "mcg_multiplier"), ("mul1", "mul1_multiplier")])
def test_foreign_multiplier_is_refused(tmp_path, name, flag):
    from safetensors.numpy import save_file
    l = _layer("m.proj", 2, 128, 128, 7)
    tensors = {"m.proj.trellis": l.trellis.view(np.int16), "m.proj.suh": l.suh, "m.proj.svh": l.svh,
               f"m.proj.{name}": np.array([0x12345679], dtype=np.int32)}
    save_file(tensors, str(tmp_path / "model.safetensors"))
    (tmp_path / "quantization_config.json").write_text(json.dumps(
        {"tensor_storage": {"m.proj": {"quant_format": "exl3", flag: True}}}))
    with pytest.raises(CheckpointError, match="multiplier"):
        load_exl3_layer(tmp_path, "m.proj")


def test_flag_without_stored_multiplier_loads(tmp_path):
    from safetensors.numpy import save_file
    l = _layer("m.proj", 2, 128, 128, 8)
    save_file({"m.proj.trellis": l.trellis.view(np.int16), "m.proj.suh": l.suh, "m.proj.svh": l.svh},
              str(tmp_path / "model.safetensors"))
    (tmp_path / "quantization_config.json").write_text(json.dumps(
        {"tensor_storage": {"m.proj": {"quant_format": "exl3", "mcg_multiplier": True}}}))
    got = load_exl3_layer(tmp_path, "m.proj")
    assert got.mcg and not got.mul1


def test_bad_packed_length(tmp_path):
    from safetensors.numpy import save_file
    save_file({"m.proj.trellis": np.zeros((8, 8, 24), dtype=np.int16)}, str(tmp_path / "model.safetensors"))
    (tmp_path / "quantization_config.json").write_text(json.dumps(
        {"tensor_storage": {"m.proj": {"quant_format": "exl3"}}}))
    with pytest.raises(CheckpointError, match="16\\*K"):
        load_exl3_layer(tmp_path, "m.proj")


def test_loaded_layer_matches_oracle_forward(tmp_path, oracle):
    """A layer that went through the directory decodes to the same weights and the same forward."""
    l = LAYERS[1]
    save_exl3_layers(tmp_path, [l])
    got = load_exl3_layer(tmp_path, l.key)
    x = np.random.default_rng(0).standard_normal((3, l.in_features)).astype(np.float16)
    cb = got.codebook_mode
    y0 = oracle.linear_forward(x, l.trellis, l.k, cb, l.suh, l.svh, l.bias)
    y1 = oracle.linear_forward(x, got.trellis, got.k, cb, got.suh, got.svh, got.bias)
    assert np.array_equal(y0.view(np.uint16), y1.view(np.uint16))


def test_partial_index_falls_back_to_scanning_the_shards(tmp_path):
    """An index that forgets tensors, or names a shard that is gone, must not lose layers: the
    shards themselves are searched, sub-directories included (ponyexl3/ref/loader.py:108-126)."""
    import shutil

    save_exl3_layers(tmp_path, LAYERS, shards=3)
    idx_path = tmp_path / "model.safetensors.index.json"
    idx = json.loads(idx_path.read_text())
    victim = LAYERS[0].key
    # 1. the index forgets every tensor of one layer
    for name in [n for n in idx["weight_map"] if n.startswith(victim + ".")]:
        del idx["weight_map"][name]
    # 2. another layer's shard moves into a sub-directory the index does not know about
    moved_key = LAYERS[2].key
    shard = idx["weight_map"][f"{moved_key}.trellis"]
    idx_path.write_text(json.dumps(idx))
    (tmp_path / "sub").mkdir()
    shutil.move(str(tmp_path / shard), str(tmp_path / "sub" / shard))
    ck = EXL3Checkpoint(tmp_path)
    assert ck.keys() == sorted(l.key for l in LAYERS)
    for l in LAYERS:
        _same(l, ck.layer(l.key))
