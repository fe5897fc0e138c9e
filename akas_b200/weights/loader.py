"""Weights from safetensors, by tensor name.

The checkpoint is checked against what the model's parts ask for before anything
is read: one ``WeightError`` lists every missing tensor, every unexpected tensor
and every wrong shape or unusable dtype (kreasof-ai/akas validates the whole
inventory before any allocation too: src/akas/models/lfm2/weights.py:340-349,
src/akas/checkpoints/safetensors.py:192-219). Operands of matrix products are held
in the compute dtype (bfloat16, or float32 on the 32-bit path); norm weights,
convolution taps and biases in float32; integer tables in int32.

A folder holds either ``model.safetensors`` or ``model.safetensors.index.json``
with its shards, which must lie inside the folder.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Tuple

import torch

_FLOAT = {"F32", "F16", "BF16", "F64"}
_INT = {"I64", "I32", "I16", "I8", "U8"}


class WeightError(ValueError):
    """The checkpoint does not hold exactly the tensors the model needs."""


class TensorIndex:
    """name -> (file, shape, dtype string) for every tensor of a model folder, read from the headers."""

    def __init__(self, folder):
        from safetensors import safe_open

        self.folder = Path(folder)
        index = self.folder / "model.safetensors.index.json"
        single = self.folder / "model.safetensors"
        if index.is_file():
            weight_map = json.loads(index.read_text()).get("weight_map", {})
            files = sorted(set(weight_map.values()))
        elif single.is_file():
            files = [single.name]
        else:
            raise FileNotFoundError(f"{self.folder}: neither model.safetensors nor model.safetensors.index.json")
        self.entries: Dict[str, Tuple[Path, Tuple[int, ...], str]] = {}
        root = self.folder.resolve()
        for name in files:
            path = (self.folder / name).resolve()
            if root not in path.parents or not path.is_file():
                raise WeightError(f"shard {name!r} is not a file inside {self.folder}")
            with safe_open(str(path), framework="pt") as f:
                for key in f.keys():
                    sl = f.get_slice(key)
                    self.entries[key] = (path, tuple(sl.get_shape()), str(sl.get_dtype()))

    def __contains__(self, name):
        return name in self.entries

    def read(self, name) -> torch.Tensor:
        from safetensors import safe_open

        path = self.entries[name][0]
        with safe_open(str(path), framework="pt") as f:
            return f.get_tensor(name)


def check_inventory(expected, index: TensorIndex) -> None:
    """Raises one WeightError naming every missing, unexpected, misshapen or mistyped tensor."""
    missing = sorted(n for n, p in expected.items() if n not in index and not p.optional)
    unexpected = sorted(n for n in index.entries if n not in expected)
    shapes, dtypes = [], []
    for name, param in expected.items():
        if name not in index:
            continue
        _, shape, dtype = index.entries[name]
        if tuple(shape) != tuple(param.shape):
            shapes.append(f"{name}: checkpoint {list(shape)}, model {list(param.shape)}")
        allowed = _INT if param.role == "table" else _FLOAT
        if dtype not in allowed:
            dtypes.append(f"{name}: {dtype} (wanted one of {sorted(allowed)})")
    if missing or unexpected or shapes or dtypes:
        lines = [f"checkpoint {index.folder} does not fit the model:"]
        for title, items in (("missing tensors", missing), ("unexpected tensors", unexpected),
                             ("wrong shapes", shapes), ("unusable dtypes", dtypes)):
            if items:
                lines.append(f"  {title} ({len(items)}):")
                lines.extend(f"    {item}" for item in items)
        raise WeightError("\n".join(lines))


def load_weights(model, folder) -> int:
    """Checks ``folder`` against ``model.params()``, loads every tensor, returns the bytes now on the device."""
    index = TensorIndex(folder)
    expected = model.params()
    check_inventory(expected, index)
    rt = model.rt
    loaded: Dict[str, torch.Tensor] = {}

    def get(name: str) -> torch.Tensor:
        if name not in loaded:
            role = expected[name].role
            target = rt.dtype if role == "matrix" else torch.int32 if role == "table" else torch.float32
            loaded[name] = index.read(name).to(device=rt.device, dtype=target).contiguous()
        return loaded[name]

    model.load(get, has=lambda name: name in index)
    return sum(t.numel() * t.element_size() for t in loaded.values())
