"""Typed model configurations and the one registry from an architecture's name to its model.

A configuration class reads the architecture's own `config.json` keys and validates them; no
size and no constant that `config.json` gives is written anywhere else. An architecture is a
triple (name, configuration class, spec builder): the spec builder turns a configuration into
a `ModelSpec` (hipinfer_b200/parts/spec.py), the list of parts the engine assembles.

The reference has neither: its configuration is the weight file's header
(src/api.cu:1062-1072, 1262-1268) and its graph is hard-wired.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields
from typing import Any, Callable, Dict, Optional, Type


class ConfigError(ValueError):
    """A config.json that is missing a key, has a wrong type, or asks for what the architecture lacks."""


_MISSING = object()


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration: the keys all of them share."""

    architecture: str

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:
        raise NotImplementedError


def take(d: Dict[str, Any], key: str, kind, default=_MISSING, *, positive=False, optional=False):
    """d[key] checked to be of `kind` (int, float, bool, str, dict); `default` when absent."""
    if key not in d or (d[key] is None and (optional or default is not _MISSING)):
        if default is _MISSING:
            if optional:
                return None
            raise ConfigError(f"config.json: key {key!r} is missing")
        return default
    v = d[key]
    if kind is float and isinstance(v, int) and not isinstance(v, bool):
        v = float(v)
    if kind is int and isinstance(v, bool) or not isinstance(v, kind):
        raise ConfigError(f"config.json: key {key!r} must be {kind.__name__}, got {v!r}")
    if positive and not v > 0:
        raise ConfigError(f"config.json: key {key!r} must be positive, got {v!r}")
    return v


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: Type[ModelConfig]
    build_spec: Callable[[ModelConfig], Any]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: Type[ModelConfig], build_spec: Callable[[ModelConfig], Any]) -> None:
    """Make `name` (the string in config.json's `architectures`) known to the framework."""
    _ARCHITECTURES[name] = Architecture(name, config_cls, build_spec)


def registered_architectures():
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    if name not in _ARCHITECTURES:
        raise ConfigError(f"architecture {name!r} is not registered; registered: {registered_architectures()}")
    return _ARCHITECTURES[name]


def config_from_dict(d: Dict[str, Any]) -> ModelConfig:
    """The typed configuration for a config.json dictionary, chosen by `architectures[0]`."""
    archs = d.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: key 'architectures' must be a non-empty list of names")
    return get_architecture(archs[0]).config_cls.from_dict(d)


def load_config(folder: str) -> ModelConfig:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{folder}: no config.json")
    with open(path) as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: must hold a JSON object")
    return config_from_dict(d)


def save_config(cfg: ModelConfig, folder: str) -> None:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f, indent=1)
