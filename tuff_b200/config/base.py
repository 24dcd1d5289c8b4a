"""Typed reading of a model folder's config.json.

An architecture's configuration class declares the keys it reads; nothing else in
the package looks at the raw dictionary.  `KeyReader` keeps track of which keys
were consumed so that a configuration can say what it ignored, and turns every
type or range fault into one `ConfigError` that names the key.
"""
from __future__ import annotations

import json
import os
from typing import Any, Iterable, Sequence


class ConfigError(ValueError):
    """A config.json that the architecture cannot be built from."""


_MISSING = object()


class KeyReader:
    """Reads typed values out of a config.json dictionary."""

    def __init__(self, raw: dict, where: str = "config.json"):
        if not isinstance(raw, dict):
            raise ConfigError(f"{where}: top level must be a JSON object")
        self.raw = raw
        self.where = where
        self.used: set[str] = set()

    def has(self, key: str) -> bool:
        return key in self.raw and self.raw[key] is not None

    def _get(self, keys: Sequence[str], default: Any) -> tuple[str, Any]:
        for k in keys:
            if self.has(k):
                self.used.add(k)
                return k, self.raw[k]
        if default is _MISSING:
            raise ConfigError(f"{self.where}: missing required key {' / '.join(keys)!s}")
        return keys[0], default

    def integer(self, *keys: str, default: Any = _MISSING, min_value: int | None = None) -> int:
        k, v = self._get(keys, default)
        if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
            raise ConfigError(f"{self.where}: key {k!r} must be an integer, found {v!r}")
        v = int(v)
        if min_value is not None and v < min_value:
            raise ConfigError(f"{self.where}: key {k!r} must be >= {min_value}, found {v}")
        return v

    def optional_integer(self, *keys: str, min_value: int | None = None) -> int | None:
        k, v = self._get(keys, None)
        if v is None:
            return None
        return self.integer(k, min_value=min_value)

    def number(self, *keys: str, default: Any = _MISSING, positive: bool = False) -> float:
        k, v = self._get(keys, default)
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: key {k!r} must be a number, found {v!r}")
        v = float(v)
        if positive and not v > 0.0:
            raise ConfigError(f"{self.where}: key {k!r} must be > 0, found {v}")
        return v

    def optional_number(self, *keys: str) -> float | None:
        k, v = self._get(keys, None)
        if v is None:
            return None
        return self.number(k)

    def boolean(self, *keys: str, default: Any = _MISSING) -> bool:
        k, v = self._get(keys, default)
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: key {k!r} must be true or false, found {v!r}")
        return v

    def string_list(self, *keys: str, default: Any = _MISSING) -> list[str] | None:
        k, v = self._get(keys, default)
        if v is None:
            return None
        if not isinstance(v, list) or not all(isinstance(s, str) for s in v):
            raise ConfigError(f"{self.where}: key {k!r} must be a list of strings, found {v!r}")
        return list(v)

    def integer_list(self, *keys: str, default: Any = _MISSING) -> list[int] | None:
        k, v = self._get(keys, default)
        if v is None:
            return None
        if not isinstance(v, list) or not all(isinstance(s, int) and not isinstance(s, bool) for s in v):
            raise ConfigError(f"{self.where}: key {k!r} must be a list of integers, found {v!r}")
        return list(v)

    def unused(self) -> list[str]:
        return sorted(k for k in self.raw if k not in self.used)


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json in the model folder")
    with open(path, "r", encoding="utf-8") as f:
        try:
            return json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None


def architecture_name(raw: dict, where: str = "config.json") -> str:
    """The model class name that config.json asks for (`architectures[0]`)."""
    archs = raw.get("architectures")
    if not isinstance(archs, list) or len(archs) < 1 or not isinstance(archs[0], str):
        raise ConfigError(f"{where}: key 'architectures' must be a list with the model class name")
    return archs[0]


def join_names(names: Iterable[str]) -> str:
    return ", ".join(sorted(names)) or "(none)"
