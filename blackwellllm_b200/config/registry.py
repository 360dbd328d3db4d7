"""One registry from an architecture's name to how its config.json becomes a model.

``register_architecture(name, parse)`` stores ``parse(raw_json) -> ModelConfig``.
``load_config`` reads ``config.json`` and dispatches on ``architectures[0]``,
falling back to ``model_type`` (the reference keys on ``model_type`` strings
only: src/core/config.cpp:81,226-227).
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, Mapping

from .specs import ModelConfig


class ConfigError(ValueError):
    """config.json is missing a key, has a bad value, or names an unsupported option."""


_ARCHITECTURES: Dict[str, Callable[[Mapping[str, Any]], ModelConfig]] = {}
_MODEL_TYPES: Dict[str, str] = {}


def register_architecture(name: str, parse: Callable[[Mapping[str, Any]], ModelConfig],
                          model_type: str | None = None) -> None:
    _ARCHITECTURES[name] = parse
    if model_type is not None:
        _MODEL_TYPES[model_type] = name


def registered_architectures() -> tuple:
    return tuple(sorted(_ARCHITECTURES))


def parse_config(raw: Mapping[str, Any]) -> ModelConfig:
    archs = raw.get("architectures") or []
    name = None
    if archs:
        if archs[0] in _ARCHITECTURES:
            name = archs[0]
        else:
            raise ConfigError(
                f"unsupported architecture {archs[0]!r}; registered: {list(registered_architectures())}")
    else:
        mt = raw.get("model_type")
        if mt in _MODEL_TYPES:
            name = _MODEL_TYPES[mt]
        else:
            raise ConfigError(
                f"config.json names no 'architectures' and model_type {mt!r} is not registered; "
                f"registered: {list(registered_architectures())}")
    return _ARCHITECTURES[name](raw)


def load_config(model_dir: str) -> ModelConfig:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {model_dir!r}")
    with open(path, "r", encoding="utf-8") as f:
        try:
            raw = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from e
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return parse_config(raw)
