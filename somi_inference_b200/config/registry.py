"""One registry from an architecture's name (config.json `architectures[0]`) to its config class.

The reference keys its registry by `model_type` and maps to a loader function
(somi_inference/models/loader.py:14-29, unknown type -> ValueError).  Here the
key is the architecture name, the value a config class with `from_dict` and
`to_model_spec`; the generic decoder is built from that spec, so registering an
architecture is one call and no engine file changes.
"""

from __future__ import annotations

import json
import os
from typing import Any, Protocol

from .spec import ModelSpec


class ArchitectureConfig(Protocol):
    architecture: str

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "ArchitectureConfig": ...
    def to_dict(self) -> dict[str, Any]: ...
    def to_model_spec(self) -> ModelSpec: ...


_ARCHITECTURES: dict[str, type] = {}


def register_architecture(name: str, config_cls: type) -> None:
    if name in _ARCHITECTURES and _ARCHITECTURES[name] is not config_cls:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = config_cls


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def supported_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def config_class_for(name: str) -> type:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ValueError(f"Unsupported architecture: {name!r}; supported: "
                         f"{supported_architectures()}") from None


def load_config(model_dir: str):
    """Read `model_dir/config.json` and return the typed config its architecture names."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"{model_dir!r} holds no config.json")
    with open(path, "r", encoding="utf-8") as f:
        raw = json.load(f)
    archs = raw.get("architectures")
    if not archs or not isinstance(archs, list):
        raise ValueError(f"{path}: no 'architectures' list; supported: {supported_architectures()}")
    return config_class_for(archs[0]).from_dict(raw)
