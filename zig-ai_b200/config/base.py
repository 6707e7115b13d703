"""Typed configuration: base class, error type and the architecture registry.

The reference has one struct for every model (`ModelConfig`, src/loader/model_config.zig:14-40),
filled from GGUF metadata (`fromGguf`, :46-131), and a string whitelist as its only registry
(`isSupportedArch`, :152-165).  Here each architecture owns a config class that reads the keys of
its own config.json, and a single registry maps the architecture's name to that class and to the
function that turns a configuration into a model description (a list of layers made from parts).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields
from typing import Any, Callable, Dict, Tuple


class ConfigError(ValueError):
    """A config.json that cannot describe a model: a missing key, a wrong type or sizes that do
    not fit together (the reference's MissingRequiredMetadata / InvalidMetadata /
    UnsupportedArchitecture, src/loader/model_config.zig:6-12)."""


_MISSING = object()


def read_key(d: Dict[str, Any], key: str, kind, default=_MISSING, where: str = "config.json"):
    """Fetch `key` from `d` as `kind` (int, float, bool, str, list); raise ConfigError otherwise."""
    if key not in d or d[key] is None:
        if default is _MISSING:
            raise ConfigError(f"{where}: required key '{key}' is missing")
        return default
    v = d[key]
    if kind is float and isinstance(v, (int, float)) and not isinstance(v, bool):
        return float(v)
    if kind is int and isinstance(v, int) and not isinstance(v, bool):
        return int(v)
    if kind is int and isinstance(v, float) and v == int(v):
        return int(v)
    if kind is bool and isinstance(v, bool):
        return v
    if kind is str and isinstance(v, str):
        return v
    if kind is list and isinstance(v, (list, tuple)):
        return list(v)
    raise ConfigError(f"{where}: key '{key}' should be {kind.__name__}, got {v!r}")


@dataclass
class ModelConfig:
    """What every architecture's configuration has in common."""
    architecture: str

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:
        raise NotImplementedError

    def field_dict(self) -> Dict[str, Any]:
        return {f.name: getattr(self, f.name) for f in fields(self)}


# architecture name -> (config class, function(config) -> ModelSpec)
_ARCHITECTURES: Dict[str, Tuple[type, Callable]] = {}


def register_architecture(name: str, config_cls: type, build_spec: Callable, replace: bool = False) -> None:
    """Add an architecture: its config class and the function that lays out its layers."""
    if name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = (config_cls, build_spec)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures():
    return sorted(_ARCHITECTURES)


def lookup_architecture(name: str) -> Tuple[type, Callable]:
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"unknown architecture '{name}'; registered: {', '.join(known_architectures()) or '(none)'}")
    return _ARCHITECTURES[name]


def architecture_name(d: Dict[str, Any], where: str = "config.json") -> str:
    archs = read_key(d, "architectures", list, where=where)
    if len(archs) != 1 or not isinstance(archs[0], str):
        raise ConfigError(f"{where}: 'architectures' should hold exactly one name, got {archs!r}")
    return archs[0]


def config_from_dict(d: Dict[str, Any], where: str = "config.json") -> ModelConfig:
    """The typed configuration for the architecture that `d` names."""
    if not isinstance(d, dict):
        raise ConfigError(f"{where}: top level should be an object")
    config_cls, _ = lookup_architecture(architecture_name(d, where))
    return config_cls.from_dict(d)


def load_config(model_dir_or_file: str) -> ModelConfig:
    path = model_dir_or_file
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json at {path}")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from e
    return config_from_dict(d, where=path)


def save_config(cfg: ModelConfig, model_dir: str) -> str:
    os.makedirs(model_dir, exist_ok=True)
    path = os.path.join(model_dir, "config.json")
    with open(path, "w", encoding="utf-8") as f:
        json.dump(cfg.to_dict(), f, indent=2)
        f.write("\n")
    return path
