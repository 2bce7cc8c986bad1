"""The registries: architecture name -> configuration class, and part kind -> part class.

`architecture_for(config_json)` dispatches on config.json's `model_type` as the
reference's loader does (src/models/registry.cpp:70-104) and lists what is supported
when nothing matches. Parts (mixers, feed-forwards, position encodings, norms, layer
arrangements) register under the `kind` string their spec carries, so a new part is one class plus one
`register_*` call, in the framework or outside it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Type

from .config.json_util import ConfigError, get_str_or


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type          # has from_json(dict), to_json() and model_spec()


_ARCHITECTURES: Dict[str, Architecture] = {}
_MIXERS: Dict[str, type] = {}
_FFNS: Dict[str, type] = {}
_POSITIONS: Dict[str, type] = {}
_NORMS: Dict[str, type] = {}
_ARRANGEMENTS: Dict[str, type] = {}


def register_architecture(name: str, config_class: type, aliases=()) -> None:
    arch = Architecture(name, config_class)
    for key in (name, *aliases):
        _ARCHITECTURES[key] = arch


def supported_architectures():
    return sorted({a.name for a in _ARCHITECTURES.values()})


def architecture_for(config_json: dict) -> Architecture:
    model_type = get_str_or(config_json, "model_type", None, "config.json")
    names = [model_type] if model_type else []
    archs = config_json.get("architectures")
    if isinstance(archs, list):
        names += [a for a in archs if isinstance(a, str)]
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    raise ConfigError(
        f"config.json: model_type {model_type!r} is not supported "
        f"(supported: {', '.join(supported_architectures())})")


def _register(table: Dict[str, type], what: str, kind: str, cls: type) -> None:
    if kind in table and table[kind] is not cls:
        raise ValueError(f"{what} kind '{kind}' is already registered to {table[kind].__name__}")
    table[kind] = cls


def _lookup(table: Dict[str, type], what: str, kind: str) -> type:
    if kind not in table:
        raise KeyError(f"no {what} of kind '{kind}' is registered (registered: {', '.join(sorted(table))})")
    return table[kind]


def register_mixer(kind: str, cls: type) -> None:
    _register(_MIXERS, "mixer", kind, cls)


def register_ffn(kind: str, cls: type) -> None:
    _register(_FFNS, "feed-forward", kind, cls)


def register_position(kind: str, cls: type) -> None:
    _register(_POSITIONS, "position encoding", kind, cls)


def register_norm(kind: str, cls: type) -> None:
    _register(_NORMS, "norm", kind, cls)


def register_arrangement(kind: str, cls: type) -> None:
    """How one layer's norms, mixer and feed-forward are wired (parts/block.py registers "pre_norm")."""
    _register(_ARRANGEMENTS, "layer arrangement", kind, cls)


def mixer_class(kind: str) -> type:
    return _lookup(_MIXERS, "mixer", kind)


def ffn_class(kind: str) -> type:
    return _lookup(_FFNS, "feed-forward", kind)


def position_class(kind: str) -> type:
    return _lookup(_POSITIONS, "position encoding", kind)


def norm_class(kind: str) -> type:
    return _lookup(_NORMS, "norm", kind)


def arrangement_class(kind: str) -> type:
    return _lookup(_ARRANGEMENTS, "layer arrangement", kind)
