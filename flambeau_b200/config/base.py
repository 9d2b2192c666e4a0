"""Typed reading of config.json.

A configuration class lists its keys as dataclass fields whose names ARE the
config.json keys; `ConfigReader` pulls them out of the parsed JSON with one
error class per way of failing, in the manner of the reference's metadata
reader (crates/models/qwen35-v2/src/config.rs:6-14, 36-110: missing key,
wrong architecture, bad value).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """Base class of every configuration failure."""


class MissingKey(ConfigError):
    def __init__(self, key: str, where: str = "config.json"):
        super().__init__(f"{where}: required key '{key}' is missing")
        self.key = key


class WrongArchitecture(ConfigError):
    def __init__(self, got: Any, want: str):
        super().__init__(f"config.json: architectures = {got!r}, this configuration class reads '{want}'")
        self.got, self.want = got, want


class BadValue(ConfigError):
    def __init__(self, key: str, value: Any, why: str):
        super().__init__(f"config.json: '{key}' = {value!r}: {why}")
        self.key, self.value = key, value


_MISSING = object()


class ConfigReader:
    """Typed access to a parsed config.json."""

    def __init__(self, raw: dict):
        if not isinstance(raw, dict):
            raise ConfigError("config.json: top level must be an object")
        self.raw = raw

    def _get(self, key, default):
        v = self.raw.get(key, _MISSING)
        if v is _MISSING or v is None:
            if default is _MISSING:
                raise MissingKey(key)
            return default
        return v

    def integer(self, key, default=_MISSING, minimum=None):
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v.is_integer():
                v = int(v)
            else:
                raise BadValue(key, v, "must be an integer")
        if minimum is not None and v < minimum:
            raise BadValue(key, v, f"must be >= {minimum}")
        return v

    def number(self, key, default=_MISSING, positive=False):
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise BadValue(key, v, "must be a number")
        v = float(v)
        if positive and not v > 0.0:
            raise BadValue(key, v, "must be > 0")
        return v

    def boolean(self, key, default=_MISSING):
        v = self._get(key, default)
        if not isinstance(v, bool):
            raise BadValue(key, v, "must be true or false")
        return v

    def string(self, key, default=_MISSING):
        v = self._get(key, default)
        if v is not None and not isinstance(v, str):
            raise BadValue(key, v, "must be a string")
        return v

    def architecture(self) -> str:
        archs = self.raw.get("architectures")
        if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
            raise MissingKey("architectures")
        return archs[0]


def read_config_json(folder_or_file) -> dict:
    p = Path(folder_or_file)
    if p.is_dir():
        p = p / "config.json"
    if not p.is_file():
        raise ConfigError(f"{p}: no such file")
    try:
        return json.loads(p.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{p}: not valid JSON ({e})") from None
