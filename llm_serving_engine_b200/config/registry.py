"""One registry from an architecture's name to its configuration class and builder.

``config.json`` names its architecture in ``architectures[0]``; the reference
checks only ``model_type == "qwen2"`` (``src/llmserve/checkpoint.py:35-36``),
which is kept as the fallback when ``architectures`` is absent.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

from .model_config import ConfigError, ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                      # has from_dict(dict)
    build_spec: Callable[[Any], ModelSpec]  # typed config -> ModelSpec
    model_types: tuple[str, ...] = ()


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class, build_spec, model_types=()) -> None:
    """Make ``name`` loadable.  ``config_class.from_dict`` parses config.json and
    ``build_spec`` turns the result into a ``ModelSpec``."""
    _ARCHITECTURES[name] = Architecture(name, config_class, build_spec, tuple(model_types))


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def resolve_architecture(values: dict[str, Any]) -> Architecture:
    names = values.get("architectures") or []
    if names:
        entry = _ARCHITECTURES.get(names[0])
        if entry is None:
            raise ConfigError(f"unknown architecture {names[0]!r}; known: {known_architectures()}")
        return entry
    model_type = values.get("model_type")
    for entry in _ARCHITECTURES.values():
        if model_type in entry.model_types:
            return entry
    raise ConfigError(
        f"config.json names no architecture (architectures={names!r}, model_type={model_type!r}); "
        f"known: {known_architectures()}"
    )


def load_config(folder_or_dict) -> tuple[Architecture, Any, ModelSpec]:
    """Read config.json (or take its dictionary) and return the architecture
    entry, the typed configuration and the model description."""
    if isinstance(folder_or_dict, dict):
        values = folder_or_dict
    else:
        path = Path(folder_or_dict)
        if path.is_dir():
            path = path / "config.json"
        if not path.exists():
            raise ConfigError(f"no config.json at {path}")
        values = json.loads(path.read_text())
    entry = resolve_architecture(values)
    config = entry.config_class.from_dict(values)
    return entry, config, entry.build_spec(config)
