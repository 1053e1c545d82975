"""One registry from the architecture's name (config.json "architectures"[0]) to its typed
configuration class.  The reference checks a ModelType enum instead
(tiny_llm/pipeline/pipeline.hpp:8-10, pipeline.cpp:30-31)."""
from __future__ import annotations

import json
import os
from typing import Dict, Type

from .errors import ConfigError

_ARCHITECTURES: Dict[str, type] = {}


def register_architecture(name: str, config_cls: type) -> None:
    """`config_cls` needs `from_dict(dict) -> config`, `to_dict()` and `model_spec() -> ModelSpec`."""
    for attr in ("from_dict", "to_dict", "model_spec"):
        if not hasattr(config_cls, attr):
            raise TypeError(f"configuration class {config_cls.__name__} lacks {attr}()")
    _ARCHITECTURES[name] = config_cls


def registered_architectures():
    return sorted(_ARCHITECTURES)


def config_class_for(name: str) -> type:
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"unknown architecture {name!r}; registered: {', '.join(registered_architectures()) or '(none)'}")
    return _ARCHITECTURES[name]


def config_from_dict(d: dict):
    archs = d.get("architectures")
    if not isinstance(archs, (list, tuple)) or not archs or not isinstance(archs[0], str):
        raise ConfigError('config.json: key "architectures" must be a non-empty list of names')
    return config_class_for(archs[0]).from_dict(d)


def load_config(model_dir: str):
    """The configuration of a model folder (its config.json), or of a config.json given by its own path."""
    path = model_dir if os.path.isfile(model_dir) else os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {model_dir}")
    with open(path) as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return config_from_dict(d)
