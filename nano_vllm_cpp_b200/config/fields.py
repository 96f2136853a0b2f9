"""Readers of single keys of a ``config.json`` that the typed configurations share: a missing key, a wrong type or a
value out of range is a ``ConfigError`` that names the key by its full path."""
from __future__ import annotations

from .model_config import ConfigError


def need(d: dict, key: str, typ, where: str, default=None, required: bool = True):
    if not isinstance(d, dict):
        raise ConfigError(f"config.json: '{where}' must be an object")
    where = f"{where}.{key}" if where else key
    if key not in d or d[key] is None:
        if required:
            raise ConfigError(f"config.json: required key '{where}' is missing")
        return default
    v = d[key]
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
            raise ConfigError(f"config.json: '{where}' must be an integer, found {v!r}")
        return int(v)
    if typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: '{where}' must be a number, found {v!r}")
        return float(v)
    if typ is str:
        if not isinstance(v, str):
            raise ConfigError(f"config.json: '{where}' must be a string, found {v!r}")
        return v
    if typ is dict:
        if not isinstance(v, dict):
            raise ConfigError(f"config.json: '{where}' must be an object")
        return v
    raise AssertionError(typ)


def positive(v: int, where: str) -> int:
    if v < 1:
        raise ConfigError(f"config.json: '{where}' must be positive, found {v}")
    return v
