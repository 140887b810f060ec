"""Typed reading of config.json values.

The reference deserialises config.json into a typed struct and reports a missing or
ill-typed key as a configuration error (crates/core/src/config.rs:183-255, 490-492);
`Reader` does the same for a Python dict and remembers which keys were looked at.
"""

from __future__ import annotations

import json
import os
from typing import Any

from ..errors import ConfigError

_MISSING = object()


class Reader:
    """Typed access to the keys of one config.json object."""

    def __init__(self, obj: dict, where: str = "config.json"):
        if not isinstance(obj, dict):
            raise ConfigError(f"{where}: top level must be a JSON object")
        self.obj = obj
        self.where = where
        self.seen: set[str] = set()

    def has(self, key: str) -> bool:
        return key in self.obj and self.obj[key] is not None

    def raw(self, key: str, default: Any = None) -> Any:
        self.seen.add(key)
        v = self.obj.get(key, default)
        return default if v is None else v

    def _get(self, key: str, default: Any):
        self.seen.add(key)
        v = self.obj.get(key, _MISSING)
        if v is _MISSING or v is None:
            if default is _MISSING:
                raise ConfigError(f"{self.where}: missing required key '{key}'")
            return _MISSING
        return v

    def integer(self, key: str, default: Any = _MISSING, minimum: int | None = None) -> int:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v.is_integer():
                v = int(v)
            else:
                raise ConfigError(f"{self.where}: '{key}' must be an integer, got {v!r}")
        if minimum is not None and v < minimum:
            raise ConfigError(f"{self.where}: '{key}' must be >= {minimum}, got {v}")
        return v

    def number(self, key: str, default: Any = _MISSING) -> float:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: '{key}' must be a number, got {v!r}")
        return float(v)

    def boolean(self, key: str, default: Any = _MISSING) -> bool:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: '{key}' must be true or false, got {v!r}")
        return v

    def string(self, key: str, default: Any = _MISSING) -> str:
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if not isinstance(v, str):
            raise ConfigError(f"{self.where}: '{key}' must be a string, got {v!r}")
        return v


def read_config_json(model_dir_or_file: str) -> dict:
    """Return the parsed config.json of a model folder (or of the file itself)."""
    path = model_dir_or_file
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            text = f.read()
    except OSError as e:
        raise ConfigError(f"cannot read {path}: {e}") from e
    try:
        obj = json.loads(text)
    except json.JSONDecodeError as e:
        raise ConfigError(f"Failed to parse config.json: {e}") from e
    if not isinstance(obj, dict):
        raise ConfigError(f"{path}: top level must be a JSON object")
    return obj
