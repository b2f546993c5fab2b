"""Read EXL3 layers from an on-disk checkpoint directory into `EXL3Layer` containers.

Same behaviour as the reference's loader (ponyexl3/ref/loader.py:84-173): a checkpoint is a
directory with ``quantization_config.json`` (per-tensor storage records; a layer belongs to
the path when its ``quant_format`` is ``"exl3"``), one or more ``*.safetensors`` shards and,
when sharded, ``model.safetensors.index.json`` with a ``weight_map``.  A layer ``key`` owns
the tensors ``key.trellis`` (required, 16-bit words ``(in/16, out/16, 16K)``), ``key.suh`` /
``key.svh`` (fp16 signs) or the legacy packed ``key.su`` / ``key.sv`` words, and an optional
``key.bias``.  K follows from the packed tile length (16K words), the codebook flags from the
storage record; stored multiplier tensors ``key.mcg`` / ``key.mul1`` must equal the constants
the kernels hard-wire (ponyexl3/mlx/model.py:261-283), anything else is refused instead of
decoded to garbage.

Only host work happens here (numpy views of the safetensors data); the device upload is the
owning module's job (`EXL3Linear`, `FusedEXL3Group`, `EXL3SwitchGLU`).
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Iterator

import numpy as np

from .layer import EXL3Layer

MCG_MULTIPLIER = 0xCBAC1FED     # ponyexl3/ref/codebook.py:14-16
MUL1_MULTIPLIER = 0x83DCD12D

_CONFIG = "quantization_config.json"
_INDEX = "model.safetensors.index.json"


class CheckpointError(ValueError):
    """The directory is not a loadable EXL3 checkpoint, or a layer in it is malformed."""


class EXL3Checkpoint:
    """An opened checkpoint directory: the storage records and the tensor-name -> shard map are
    read once, tensors are fetched lazily per layer."""

    def __init__(self, model_dir: str | Path):
        self.root = Path(model_dir)
        cfg_path = self.root / _CONFIG
        if not cfg_path.is_file():
            raise CheckpointError(f"{cfg_path} not found")
        with open(cfg_path) as f:
            cfg = json.load(f)
        if "quantization_config" in cfg and "tensor_storage" not in cfg:
            cfg = cfg["quantization_config"]      # the record may sit inside a model config.json
        self.storage: dict[str, dict] = {
            key: rec for key, rec in cfg.get("tensor_storage", {}).items()
            if isinstance(rec, dict) and rec.get("quant_format") == "exl3"}
        # tensor name -> shard.  The index file is taken where it holds good; a tensor it does not
        # list, or whose shard is missing, is looked for in the shards themselves (top level, then
        # sub-directories), as the reference does (ponyexl3/ref/loader.py:108-126).
        self._where: dict[str, Path] = {}
        idx_path = self.root / _INDEX
        if idx_path.is_file():
            with open(idx_path) as f:
                for name, shard in json.load(f).get("weight_map", {}).items():
                    path = self.root / shard
                    if path.is_file():
                        self._where[name] = path
        from safetensors import safe_open
        found = sorted(self.root.glob("*.safetensors")) + sorted(
            p for p in self.root.glob("**/*.safetensors") if p.parent != self.root)
        for shard in found:
            with safe_open(str(shard), framework="np") as f:
                for name in f.keys():
                    self._where.setdefault(name, shard)
        self._open: dict[Path, object] = {}

    # -- tensor access ---------------------------------------------------------------------
    def _handle(self, shard: Path):
        h = self._open.get(shard)
        if h is None:
            from safetensors import safe_open
            if not shard.is_file():
                raise CheckpointError(f"shard {shard} named by the index is missing")
            h = safe_open(str(shard), framework="np")
            self._open[shard] = h
        return h

    def has(self, name: str) -> bool:
        return name in self._where

    def tensor(self, name: str) -> np.ndarray | None:
        shard = self._where.get(name)
        return None if shard is None else self._handle(shard).get_tensor(name)

    # -- layers ----------------------------------------------------------------------------
    def keys(self) -> list[str]:
        """Layer keys with an exl3 storage record whose trellis is present, sorted."""
        return sorted(k for k in self.storage if self.has(f"{k}.trellis"))

    def __contains__(self, key: str) -> bool:
        return key in self.storage and self.has(f"{key}.trellis")

    def layer(self, key: str) -> EXL3Layer:
        rec = self.storage.get(key)
        if rec is None:
            raise CheckpointError(f"{key}: no exl3 storage record in {_CONFIG}")
        trellis = self.tensor(f"{key}.trellis")
        if trellis is None:
            raise CheckpointError(f"{key}: tensor {key}.trellis not found in any shard")
        if trellis.ndim != 3 or trellis.dtype.itemsize != 2:
            raise CheckpointError(f"{key}: trellis must be 3-D 16-bit words, got "
                                  f"{trellis.dtype} {trellis.shape}")
        trellis = np.ascontiguousarray(trellis).view(np.uint16)
        in_tiles, out_tiles, packed = trellis.shape
        if packed % 16 or not 1 <= packed // 16 <= 8:
            raise CheckpointError(f"{key}: packed tile length {packed} is not 16*K, K in 1..8")
        mcg, mul1 = bool(rec.get("mcg_multiplier")), bool(rec.get("mul1_multiplier"))
        if mcg:
            self._check_multiplier(key, "mcg", MCG_MULTIPLIER)
        if mul1:
            self._check_multiplier(key, "mul1", MUL1_MULTIPLIER)
        layer = EXL3Layer(
            key=key, in_features=in_tiles * 16, out_features=out_tiles * 16, k=packed // 16,
            trellis=trellis, suh=self._signs(key, "suh", "su", in_tiles * 16),
            svh=self._signs(key, "svh", "sv", out_tiles * 16), bias=self._f16(f"{key}.bias"),
            mcg=mcg, mul1=mul1)
        layer.validate()
        return layer

    def layers(self) -> Iterator[EXL3Layer]:
        for key in self.keys():
            yield self.layer(key)

    # -- helpers ---------------------------------------------------------------------------
    def _f16(self, name: str) -> np.ndarray | None:
        t = self.tensor(name)
        return None if t is None else np.ascontiguousarray(t).astype(np.float16, copy=False)

    def _signs(self, key: str, name16: str, name_packed: str, n: int) -> np.ndarray | None:
        """fp16 sign vector if stored, else the legacy packed words (kept packed: the owning
        module expands them at upload), else None."""
        t = self._f16(f"{key}.{name16}")
        if t is not None:
            if t.shape != (n,):
                raise CheckpointError(f"{key}.{name16}: shape {t.shape} != ({n},)")
            return t
        p = self.tensor(f"{key}.{name_packed}")
        if p is None:
            return None
        if p.dtype.itemsize != 2 or p.size != n // 16:
            raise CheckpointError(f"{key}.{name_packed}: expected {n // 16} 16-bit sign words")
        return np.ascontiguousarray(p).reshape(-1).view(np.int16)

    def _check_multiplier(self, key: str, name: str, expected: int) -> None:
        t = self.tensor(f"{key}.{name}")
        if t is None:
            return
        got = int(np.asarray(t).reshape(-1)[0].astype(np.int64)) & 0xFFFFFFFF
        if got != expected:
            raise CheckpointError(
                f"{key}: stored {name} multiplier {got:#x} != supported {expected:#x}")


# -- function-style surface, the names the reference exports (ponyexl3/ref/loader.py) ----------

def list_exl3_layers(model_dir: str | Path) -> list[str]:
    return EXL3Checkpoint(model_dir).keys()


def has_exl3_layer_weights(model_dir: str | Path, key: str) -> bool:
    return key in EXL3Checkpoint(model_dir)


def load_exl3_layer(model_dir: str | Path, key: str) -> EXL3Layer:
    return EXL3Checkpoint(model_dir).layer(key)


def save_exl3_layers(model_dir: str | Path, layers: list[EXL3Layer], shards: int = 1) -> None:
    """Write `layers` as a checkpoint directory in the layout above (tests and synthetic
    benchmarks use it; the converter that produces real checkpoints is a different product)."""
    from safetensors.numpy import save_file
    root = Path(model_dir)
    root.mkdir(parents=True, exist_ok=True)
    storage, per_shard = {}, [dict() for _ in range(max(1, shards))]
    for i, l in enumerate(layers):
        l.validate()
        rec = {"quant_format": "exl3", "bits_per_weight": l.k}
        t = per_shard[i % len(per_shard)]
        t[f"{l.key}.trellis"] = np.ascontiguousarray(l.trellis).view(np.int16)
        if l.mcg:
            rec["mcg_multiplier"] = True
            t[f"{l.key}.mcg"] = np.array([MCG_MULTIPLIER], dtype=np.uint32).view(np.int32)
        if l.mul1:
            rec["mul1_multiplier"] = True
            t[f"{l.key}.mul1"] = np.array([MUL1_MULTIPLIER], dtype=np.uint32).view(np.int32)
        for attr, packed_name in (("suh", "su"), ("svh", "sv")):
            v = getattr(l, attr)
            if v is not None:
                is_f = v.dtype in (np.float16, np.float32)
                t[f"{l.key}.{attr if is_f else packed_name}"] = (
                    v.astype(np.float16) if is_f else np.ascontiguousarray(v).view(np.int16))
        if l.bias is not None:
            t[f"{l.key}.bias"] = l.bias.astype(np.float16)
        storage[l.key] = rec
    with open(root / _CONFIG, "w") as f:
        json.dump({"quant_method": "exl3", "tensor_storage": storage}, f, indent=1)
    if len(per_shard) == 1:
        save_file(per_shard[0], str(root / "model.safetensors"))
        return
    weight_map = {}
    for i, t in enumerate(per_shard):
        fname = f"model-{i + 1:05d}-of-{len(per_shard):05d}.safetensors"
        save_file(t, str(root / fname))
        weight_map.update({name: fname for name in t})
    with open(root / _INDEX, "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f, indent=1)
