"""One registry from the architecture's name (config.json "architectures"[0]) to its model.

The reference keeps a dict SUPPORTED and a describe() that refuses unknown names with the
list of supported ones (engine/models.py:1-15).  An entry here is a pair: the typed
configuration class and the function that turns a configuration into a ModelSpec.
"""
from __future__ import annotations

from typing import Callable, Dict, NamedTuple

from .model_config import ConfigError, read_config_json


class Architecture(NamedTuple):
    name: str
    description: str
    config_class: type
    build_spec: Callable


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, description: str, config_class: type, build_spec: Callable) -> None:
    _ARCHITECTURES[name] = Architecture(name, description, config_class, build_spec)


def supported_architectures() -> Dict[str, str]:
    _load_builtin()
    return {a.name: a.description for a in _ARCHITECTURES.values()}


def resolve(raw_config: dict) -> Architecture:
    _load_builtin()
    archs = raw_config.get("architectures") or []
    if not archs:
        raise ConfigError("config.json has no 'architectures' entry")
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(f"architecture '{name}' is not supported. Supported: {', '.join(sorted(_ARCHITECTURES))}")
    return _ARCHITECTURES[name]


def load_config(model_dir: str):
    """(typed config, ModelSpec) of a model folder, the class chosen by config.json."""
    raw = read_config_json(model_dir)
    arch = resolve(raw)
    cfg = arch.config_class.from_dict(raw)
    return cfg, arch.build_spec(cfg)


def _load_builtin():
    from .. import models  # noqa: F401  (registers the built-in architectures)
