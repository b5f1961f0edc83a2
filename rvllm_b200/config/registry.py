"""One registry from an architecture's name to its configuration type and its model.

config.json's `architectures[0]` picks the entry, before any weight is read, as the
reference matches GGUF's `general.architecture` first (src/weights.rs:88-100,
303-309).  An entry holds the typed configuration class and the function that turns
a configuration into a `ModelSpec`; the generic `Model` runs every spec.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict

from ..errors import ConfigError
from .base import read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any            # has from_dict(data, where) and to_dict()
    build_spec: Callable         # config -> ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class, build_spec, replace: bool = False):
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_class, build_spec)
    return _ARCHITECTURES[name]


def registered_architectures():
    return sorted(_ARCHITECTURES)


def architecture(name: str) -> Architecture:
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unsupported architecture {name!r} "
                          f"(supported: {', '.join(registered_architectures())})")
    return _ARCHITECTURES[name]


def config_from_dict(data: Dict[str, Any], where: str = "config.json"):
    archs = data.get("architectures") if isinstance(data, dict) else None
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError(f"{where}: missing key 'architectures' (a list naming the model class)")
    return architecture(archs[0]).config_class.from_dict(data, where)


def load_config(folder: str):
    """The typed configuration of a model folder."""
    import os
    return config_from_dict(read_config_json(folder), os.path.join(folder, "config.json"))
