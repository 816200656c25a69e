"""One registry from an architecture's name (config.json `architectures[0]`) to
its configuration class.  The configuration class turns config.json into a
`ModelPlan`; the model is then built from that plan by `parts.model.build_model`.

The reference has no registry: src/main.cpp:158 builds Qwen3ForCausalLM
unconditionally and only prints `model_type`.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Type

_ARCHITECTURES: Dict[str, type] = {}


class ConfigError(ValueError):
    """config.json is missing a key, holds a bad value, or asks for what is not built."""


def register_architecture(name: str) -> Callable[[type], type]:
    """Class decorator: `name` is the string config.json carries in `architectures`.

    The class must offer `from_dict(d) -> config`, `to_dict() -> d` and
    `plan() -> ModelPlan`.
    """
    def deco(cls: type) -> type:
        for attr in ("from_dict", "to_dict", "plan"):
            if not hasattr(cls, attr):
                raise TypeError(f"{cls.__name__} lacks {attr}()")
        _ARCHITECTURES[name] = cls
        cls.architecture = name
        return cls
    return deco


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures():
    return sorted(_ARCHITECTURES)


def config_class_for(name: str) -> type:
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"unknown architecture {name!r}; registered: {', '.join(registered_architectures()) or '(none)'}")
    return _ARCHITECTURES[name]


def config_from_dict(d: dict):
    archs = d.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("Missing required config field: architectures")
    return config_class_for(archs[0]).from_dict(d)


def load_config(model_dir: str):
    """Read `<model_dir>/config.json` and return the typed configuration its
    `architectures[0]` names."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"Failed to open config file: {path}")
    with open(path, "r", encoding="utf-8") as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return config_from_dict(d)


def save_config(config, model_dir: str) -> None:
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=2)
        f.write("\n")
