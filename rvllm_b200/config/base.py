"""Typed reading of config.json keys.

`Reader` wraps the parsed JSON object and gives each key through a typed accessor
that names the key in its error, the way the reference names a GGUF metadata key
that is missing or of the wrong type (src/weights.rs:13-36).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional

from ..errors import ConfigError

_MISSING = object()


class Reader:
    def __init__(self, data: Dict[str, Any], where: str = "config.json"):
        if not isinstance(data, dict):
            raise ConfigError(f"{where}: expected a JSON object")
        self.data = data
        self.where = where

    def _get(self, key: str, default):
        if key in self.data and self.data[key] is not None:
            return self.data[key]
        if default is _MISSING:
            raise ConfigError(f"{self.where}: missing key {key!r}")
        return default

    def has(self, key: str) -> bool:
        return key in self.data and self.data[key] is not None

    def int(self, key: str, default=_MISSING, minimum: Optional[int] = None) -> int:
        v = self._get(key, default)
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"{self.where}: key {key!r} must be an integer, got {v!r}")
        if minimum is not None and v < minimum:
            raise ConfigError(f"{self.where}: key {key!r} must be at least {minimum}, got {v}")
        return v

    def float(self, key: str, default=_MISSING) -> float:
        v = self._get(key, default)
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: key {key!r} must be a number, got {v!r}")
        return float(v)

    def optional_float(self, key: str) -> Optional[float]:
        return self.float(key) if self.has(key) else None

    def optional_int(self, key: str, minimum: Optional[int] = None) -> Optional[int]:
        return self.int(key, minimum=minimum) if self.has(key) else None

    def bool(self, key: str, default=_MISSING) -> bool:
        v = self._get(key, default)
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: key {key!r} must be true or false, got {v!r}")
        return v

    def str(self, key: str, default=_MISSING) -> str:
        v = self._get(key, default)
        if not isinstance(v, str):
            raise ConfigError(f"{self.where}: key {key!r} must be a string, got {v!r}")
        return v

    def int_list(self, key: str, default=_MISSING) -> List[int]:
        v = self._get(key, default)
        if not isinstance(v, list) or any(isinstance(x, bool) or not isinstance(x, int) for x in v):
            raise ConfigError(f"{self.where}: key {key!r} must be a list of integers, got {v!r}")
        return list(v)

    def str_list(self, key: str, default=_MISSING) -> List[str]:
        v = self._get(key, default)
        if not isinstance(v, list) or any(not isinstance(x, str) for x in v):
            raise ConfigError(f"{self.where}: key {key!r} must be a list of strings, got {v!r}")
        return list(v)


def read_config_json(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{folder}: no config.json in this model folder")
    with open(path) as f:
        try:
            return json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
