"""One registry from an architecture's name to its configuration class and its model.

vt-transformer picks a model by which graph file is passed to the binary
(v1/models/qwen2-7b/chat.cpp:204-231); here config.json's ``architectures[0]`` picks
an ``Architecture``: the class that reads config.json and a function that turns the
configuration into a ``ModelSpec`` (pure data: which parts, of which sizes, in which
order).  Adding an architecture is one ``register_architecture`` call; nothing else in
the package names a model.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Type

from .base import ConfigError, ModelConfig, architecture_name, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Type[ModelConfig]
    model_spec: Callable[[ModelConfig], "object"]   # ModelConfig -> parts.specs.ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Type[ModelConfig],
                          model_spec: Callable[[ModelConfig], "object"], replace: bool = False) -> Architecture:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{name}' is registered already")
    arch = Architecture(name, config_class, model_spec)
    _ARCHITECTURES[name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures():
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"architecture '{name}' is not registered; known: {', '.join(known_architectures()) or 'none'}") from None


def config_from_dict(data, where: str = "config.json") -> ModelConfig:
    arch = get_architecture(architecture_name(data, where))
    return arch.config_class.from_dict(data, where)


def load_config(folder: str) -> ModelConfig:
    """Reads ``folder/config.json`` with the configuration class its architecture names."""
    import os
    return config_from_dict(read_config_json(folder), os.path.join(folder, "config.json"))
