"""One registry from an architecture's name (``config.json`` ``architectures[0]``)
to its typed configuration class.

The reference imports ``Qwen2ForCausalLM`` directly (v10_triton_paged_gqa/llm.py:15)
and reads its configuration as a raw dict (v10_triton_paged_gqa/llm.py:38); a registry
replaces the import so that another architecture is one ``register_architecture`` call.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Callable, Protocol


class ArchitectureConfig(Protocol):
    """What a typed configuration must offer."""

    @classmethod
    def from_dict(cls, raw: dict) -> "ArchitectureConfig": ...

    def to_dict(self) -> dict: ...

    def model_spec(self): ...


_ARCHITECTURES: dict[str, type] = {}


def register_architecture(name: str, config_cls: type | None = None) -> Callable | None:
    """Register ``config_cls`` under ``name``; usable as a decorator."""

    def _register(cls: type) -> type:
        _ARCHITECTURES[name] = cls
        return cls

    if config_cls is None:
        return _register
    _register(config_cls)
    return None


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def config_class_for(name: str) -> type:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise KeyError(
            f"unknown architecture {name!r}; registered: {', '.join(known_architectures()) or 'none'}"
        ) from None


def config_from_dict(raw: dict):
    archs = raw.get("architectures")
    if not isinstance(archs, (list, tuple)) or not archs:
        raise ValueError("config.json has no 'architectures' list to choose the model by")
    return config_class_for(archs[0]).from_dict(raw)


def load_config(model_dir: str | Path):
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"no config.json in {model_dir}")
    return config_from_dict(json.loads(path.read_text()))
