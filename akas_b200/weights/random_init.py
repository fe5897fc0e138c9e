"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a configuration and a seed.

Matrices and convolution taps are N(0, std), norm weights 1 + N(0, std), biases
N(0, std); std defaults to 0.02. Values are drawn on the CPU in float32, tensor by
tensor in the order of the model's own inventory, so a seed gives the same model
everywhere; they are then stored in ``dtype``. kreasof-ai/akas has no such mode in
its engine; its test fixture draws N(0, 0.015) matrices and all-ones norm weights
(tests/support/diagnostic.py:98-116).
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from ..models.decoder import Decoder
from ..parts.base import Runtime

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def random_tensors(config, seed: int, std: float = 0.02, dtype: str = "bfloat16") -> dict:
    spec = config.model_spec()
    model = Decoder(spec, Runtime(torch.float32, torch.device("cpu"), ops=None))
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    store = _DTYPES[dtype]
    out = {}
    for name, param in model.params().items():
        if param.optional:
            continue
        if param.role == "table":
            raise ValueError(f"{name}: no rule for a random integer table")
        value = torch.randn(param.shape, generator=gen, dtype=torch.float32) * std + param.mean
        out[name] = value.to(store).contiguous()
    return out


def write_random_model(folder, config, seed: int, std: float = 0.02, dtype: str = "bfloat16") -> Path:
    """Creates ``folder`` with config.json and model.safetensors; returns the folder."""
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    data = config.to_dict()
    data["torch_dtype"] = dtype
    (folder / "config.json").write_text(json.dumps(data, indent=2) + "\n")
    save_file(random_tensors(config, seed, std, dtype), str(folder / "model.safetensors"))
    return folder
