"""Typed getters over a parsed config.json, each failing with the key's name.

The reference reads config.json through helpers that name the file and the key in
every error (src/models/config_util.cpp:16-66); these do the same for Python dicts.
"""
from __future__ import annotations

import json
import os
from typing import Any, List, Optional


class ConfigError(ValueError):
    """A config.json that cannot be turned into a typed configuration."""


def read_json(path: str) -> dict:
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: file not found")
    with open(path, "r", encoding="utf-8") as f:
        try:
            obj = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(obj, dict):
        raise ConfigError(f"{path}: the top level must be an object")
    return obj


def _need(obj: dict, key: str, where: str) -> Any:
    if key not in obj or obj[key] is None:
        raise ConfigError(f"{where}: missing '{key}'")
    return obj[key]


def get_int(obj: dict, key: str, where: str) -> int:
    v = _need(obj, key, where)
    if isinstance(v, bool) or not isinstance(v, int):
        if isinstance(v, float) and v == int(v):
            return int(v)
        raise ConfigError(f"{where}: '{key}' must be an integer, got {v!r}")
    return v


def get_int_or(obj: dict, key: str, default: int, where: str) -> int:
    if key not in obj or obj[key] is None:
        return default
    return get_int(obj, key, where)


def get_float(obj: dict, key: str, where: str) -> float:
    v = _need(obj, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"{where}: '{key}' must be a number, got {v!r}")
    return float(v)


def get_float_or(obj: dict, key: str, default: float, where: str) -> float:
    if key not in obj or obj[key] is None:
        return default
    return get_float(obj, key, where)


def get_bool_or(obj: dict, key: str, default: bool, where: str) -> bool:
    if key not in obj or obj[key] is None:
        return default
    v = obj[key]
    if not isinstance(v, bool):
        raise ConfigError(f"{where}: '{key}' must be true or false, got {v!r}")
    return v


def get_str(obj: dict, key: str, where: str) -> str:
    v = _need(obj, key, where)
    if not isinstance(v, str):
        raise ConfigError(f"{where}: '{key}' must be a string, got {v!r}")
    return v


def get_str_or(obj: dict, key: str, default: Optional[str], where: str) -> Optional[str]:
    if key not in obj or obj[key] is None:
        return default
    return get_str(obj, key, where)


def get_int_list(obj: dict, key: str, where: str) -> List[int]:
    """An integer or a list of integers; absent gives an empty list
    (eos_token_id is written both ways, src/models/config_util.cpp:137-147)."""
    if key not in obj or obj[key] is None:
        return []
    v = obj[key]
    if isinstance(v, int) and not isinstance(v, bool):
        return [v]
    if isinstance(v, list) and all(isinstance(x, int) and not isinstance(x, bool) for x in v):
        return list(v)
    raise ConfigError(f"{where}: '{key}' must be an integer or a list of integers, got {v!r}")
