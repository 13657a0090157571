"""One registry from an architecture's name to its model description.

The reference keeps a singleton name -> factory map
(src/model/model_registry.cpp:5-24) and registers "llama", "qwen" and "gemma"
in Engine::initialize (src/core/engine.cpp:26-28); an unknown name yields
"Unknown model architecture" (src/core/engine.cpp:40-44).  Here a registered
architecture is a function ``config.json dict -> (typed config, ModelSpec)``;
the engine builds the model from the ModelSpec alone.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Tuple

from .engine_config import ConfigError
from .model_spec import ModelSpec

_ARCHITECTURES: Dict[str, Callable[[dict], Tuple[object, ModelSpec]]] = {}


def register_architecture(*names: str):
    """Decorator: register ``fn(config_dict) -> (typed_config, ModelSpec)`` under ``names``."""
    def deco(fn):
        for n in names:
            _ARCHITECTURES[n] = fn
        return fn
    return deco


def known_architectures():
    return sorted(_ARCHITECTURES)


def read_config_json(model_path: str) -> dict:
    path = os.path.join(model_path, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"Cannot open config: {path}")
    with open(path, "r") as f:
        try:
            cfg = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path} is not valid JSON: {e}") from None
    if not isinstance(cfg, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return cfg


def resolve_architecture(config: dict, model_arch: str = "") -> Tuple[object, ModelSpec]:
    """Pick the architecture (``model_arch`` if given, else ``architectures[0]``) and build its spec."""
    name = model_arch
    if not name:
        archs = config.get("architectures")
        if not (isinstance(archs, list) and archs and isinstance(archs[0], str)):
            raise ConfigError(
                "config.json has no 'architectures' list and no model_arch was given; "
                f"known architectures: {known_architectures()}")
        name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(f"Unknown model architecture: {name!r}; known: {known_architectures()}")
    typed, spec = _ARCHITECTURES[name](config)
    spec.validate()
    return typed, spec
