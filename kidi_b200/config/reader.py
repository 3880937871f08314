"""Typed access to the keys of a config.json.

The reference keeps its configuration as an untyped YAML node and lets a missing
key throw, which it reports as INVALID_MANIFEST (src/kidi/model/qwen3.cpp:38-67).
Here every architecture owns a typed, frozen dataclass instead; this reader is the
only place that touches the raw dictionary, and it turns a missing key or a value
of the wrong type into the same INVALID_MANIFEST error, naming the key.
"""
from __future__ import annotations

import json
import math
import os
from typing import Any, Mapping, Optional, Sequence

from ..errors import invalid_manifest, io_error

_MISSING = object()


class ConfigReader:
    """Reads keys of one JSON object and remembers which ones were asked for."""

    def __init__(self, values: Mapping[str, Any], where: str = "config.json"):
        if not isinstance(values, Mapping):
            raise invalid_manifest(f"{where} must hold a JSON object")
        self._values = values
        self._where = where

    def has(self, key: str) -> bool:
        return key in self._values and self._values[key] is not None

    def _get(self, key: str, default: Any) -> Any:
        value = self._values.get(key, _MISSING)
        if value is _MISSING or value is None:
            if default is _MISSING:
                raise invalid_manifest(f"{self._where}: missing key '{key}'")
            return default
        return value

    def integer(self, key: str, default: Any = _MISSING) -> int:
        value = self._get(key, default)
        if isinstance(value, bool) or not isinstance(value, int):
            if isinstance(value, float) and value.is_integer():
                return int(value)
            raise invalid_manifest(f"{self._where}: '{key}' must be an integer, found {value!r}")
        return value

    def number(self, key: str, default: Any = _MISSING) -> float:
        value = self._get(key, default)
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise invalid_manifest(f"{self._where}: '{key}' must be a number, found {value!r}")
        value = float(value)
        if not math.isfinite(value):
            raise invalid_manifest(f"{self._where}: '{key}' must be finite")
        return value

    def string(self, key: str, default: Any = _MISSING) -> str:
        value = self._get(key, default)
        if not isinstance(value, str):
            raise invalid_manifest(f"{self._where}: '{key}' must be a string, found {value!r}")
        return value

    def boolean(self, key: str, default: Any = _MISSING) -> bool:
        value = self._get(key, default)
        if not isinstance(value, bool):
            raise invalid_manifest(f"{self._where}: '{key}' must be true or false, found {value!r}")
        return value

    def strings(self, key: str, default: Any = _MISSING) -> Optional[Sequence[str]]:
        value = self._get(key, default)
        if value is None:
            return None
        if not isinstance(value, (list, tuple)) or not all(isinstance(item, str) for item in value):
            raise invalid_manifest(f"{self._where}: '{key}' must be a list of strings")
        return tuple(value)

    def child(self, key: str) -> Optional["ConfigReader"]:
        value = self._values.get(key)
        if value is None:
            return None
        if not isinstance(value, Mapping):
            raise invalid_manifest(f"{self._where}: '{key}' must be an object")
        return ConfigReader(value, f"{self._where}:{key}")

    def raw(self, key: str, default: Any = None) -> Any:
        return self._values.get(key, default)


def read_config_json(model_dir: str) -> dict:
    """Loads `<model_dir>/config.json` (the folder contract of
    src/kidi/checkpoint/config.cpp:234-256: one directory, one config.json)."""
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as handle:
            values = json.load(handle)
    except FileNotFoundError:
        raise io_error(f"no config.json in {model_dir}") from None
    except OSError as error:
        raise io_error(f"cannot read {path}: {error}") from None
    except json.JSONDecodeError as error:
        raise invalid_manifest(f"{path} is not valid JSON: {error}") from None
    if not isinstance(values, dict):
        raise invalid_manifest(f"{path} must hold a JSON object")
    return values
