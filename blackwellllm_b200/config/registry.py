"""One registry from an architecture's name to how its config.json becomes a model.

``register_architecture(name, parse)`` stores ``parse(raw_json) -> ModelConfig``.
``load_config`` reads ``config.json`` and dispatches on ``architectures[0]``,
falling back to ``model_type`` (the reference keys on ``model_type`` strings
only: src/core/config.cpp:81,226-227); end-of-sequence ids that a
``generation_config.json`` in the same folder lists are added to config.json's.
"""
from __future__ import annotations

import dataclasses
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
    cfg = parse_config(raw)
    extra = _generation_eos(model_dir)
    if extra:
        merged = tuple(dict.fromkeys(tuple(extra) + tuple(cfg.eos_token_ids)))
        cfg = dataclasses.replace(cfg, eos_token_ids=merged)
    return cfg


def _generation_eos(model_dir: str) -> tuple:
    """End-of-sequence ids of ``generation_config.json`` beside config.json, if that file is there
    (a checkpoint may list several there and only one, or none, in config.json).  They come first,
    then those of config.json that are not among them."""
    path = os.path.join(model_dir, "generation_config.json")
    if not os.path.isfile(path):
        return ()
    with open(path, "r", encoding="utf-8") as f:
        try:
            gen = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from e
    eos = gen.get("eos_token_id") if isinstance(gen, dict) else None
    if eos is None:
        return ()
    ids = [eos] if isinstance(eos, int) and not isinstance(eos, bool) else eos
    if not isinstance(ids, (list, tuple)) or not all(isinstance(i, int) and not isinstance(i, bool) and i >= 0 for i in ids):
        raise ConfigError(f"{path}: 'eos_token_id' must be a non-negative integer or a list of them, got {eos!r}")
    return tuple(ids)
