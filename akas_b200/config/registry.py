"""One registry from an architecture's name to its typed configuration.

``config.json["architectures"][0]`` (or, failing that, ``model_type``) picks the
entry. The configuration class must offer ``from_dict(mapping)``, ``to_dict()``
and ``model_spec() -> ModelSpec``; the engine builds every architecture from its
``ModelSpec`` with the same generic decoder, so registering a configuration class
is all that a new architecture made of existing parts needs.

kreasof-ai/akas finds its model declarations by a package walk and takes
``--definition module:Class`` on the command line (src/akas/models/__init__.py:4-19,
src/akas/cli.py:157-165); here the model folder names its own architecture.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Dict, Mapping

_ARCHITECTURES: Dict[str, type] = {}
_MODEL_TYPES: Dict[str, str] = {}


def register_architecture(name: str, config_class: type, model_type: str | None = None) -> None:
    for attr in ("from_dict", "model_spec"):
        if not hasattr(config_class, attr):
            raise TypeError(f"{config_class.__name__} lacks {attr}()")
    _ARCHITECTURES[name] = config_class
    if model_type is not None:
        _MODEL_TYPES[model_type] = name


def architectures() -> tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def architecture_of(data: Mapping[str, Any]) -> str:
    names = data.get("architectures") or []
    for name in names:
        if name in _ARCHITECTURES:
            return name
    model_type = data.get("model_type")
    if model_type in _MODEL_TYPES:
        return _MODEL_TYPES[model_type]
    raise KeyError(
        f"no registered architecture for architectures={list(names)!r}, model_type={model_type!r}; "
        f"registered: {list(architectures())}"
    )


def config_from_dict(data: Mapping[str, Any]):
    return _ARCHITECTURES[architecture_of(data)].from_dict(data)


def load_config(folder):
    """The typed configuration of the model in ``folder`` (or of a config.json path)."""
    path = Path(folder)
    if path.is_dir():
        path = path / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"{path}: no config.json")
    return config_from_dict(json.loads(path.read_text()))
