"""Typed model configurations read from a model folder's config.json.

vt-transformer has no such layer: its sizes are literals at the top of each graph
file (v1/models/qwen2-7b/inference_fp16.dag:1-14) and again in
v1/models/qwen2-7b/memory.hpp:3-7.  Here every size and constant comes from
config.json through a ``KeyReader`` that names the key in every error, and an
architecture's configuration class says which keys it has.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass
from typing import Any, Dict, Optional


class ConfigError(ValueError):
    """config.json is missing a key, or a key has a value the engine cannot run."""


_MISSING = object()


class KeyReader:
    """Reads typed values out of a parsed config.json and records which keys were read."""

    def __init__(self, data: Dict[str, Any], where: str = "config.json"):
        if not isinstance(data, dict):
            raise ConfigError(f"{where}: expected a JSON object, found {type(data).__name__}")
        self.data = data
        self.where = where
        self.read = set()

    def _get(self, key: str, default):
        self.read.add(key)
        if key in self.data and self.data[key] is not None:
            return self.data[key]
        if default is _MISSING:
            raise ConfigError(f"{self.where}: key '{key}' is required and missing")
        return default

    def integer(self, key: str, default=_MISSING, minimum: Optional[int] = None) -> Optional[int]:
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v == int(v):
                v = int(v)
            else:
                raise ConfigError(f"{self.where}: key '{key}' must be an integer, found {v!r}")
        if minimum is not None and v < minimum:
            raise ConfigError(f"{self.where}: key '{key}' must be at least {minimum}, found {v}")
        return v

    def number(self, key: str, default=_MISSING, positive: bool = False) -> Optional[float]:
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: key '{key}' must be a number, found {v!r}")
        if positive and not v > 0:
            raise ConfigError(f"{self.where}: key '{key}' must be positive, found {v}")
        return float(v)

    def boolean(self, key: str, default=_MISSING) -> bool:
        v = self._get(key, default)
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: key '{key}' must be true or false, found {v!r}")
        return v

    def string(self, key: str, default=_MISSING) -> Optional[str]:
        v = self._get(key, default)
        if v is not None and not isinstance(v, str):
            raise ConfigError(f"{self.where}: key '{key}' must be a string, found {v!r}")
        return v

    def raw(self, key: str, default=_MISSING):
        return self._get(key, default)


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration.  ``architecture`` is the registry key
    (config.json's ``architectures[0]``)."""

    architecture: str

    @classmethod
    def from_dict(cls, data: Dict[str, Any], where: str = "config.json") -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:
        """The config.json that ``from_dict`` reads back to an equal configuration."""
        d = asdict(self)
        arch = d.pop("architecture")
        d = {k: v for k, v in d.items() if v is not None}
        d["architectures"] = [arch]
        return d

    def save(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(self.to_dict(), f, indent=2)


def read_config_json(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no such file (a model folder holds config.json and model.safetensors)")
    with open(path) as f:
        try:
            return json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from None


def architecture_name(data: Dict[str, Any], where: str = "config.json") -> str:
    archs = data.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError(f"{where}: key 'architectures' must be a list that names the model class")
    return archs[0]
