"""The one registry from an architecture's name to its model.

The reference promises a per-architecture table (mynah-slm src/model.h:3-5)
but links its only architecture directly (cli/main.c:8). Here the name in
config.json's `architectures[0]` selects an `Architecture`: a function from
config.json (and generation_config.json, when the folder has one) to a typed
config. The typed config yields the architecture-neutral `ModelSpec` that
weights, cache and engine are built from, and the config.json it is read back
from (used by the random-weights writer).

Adding an architecture is one `register_architecture` call; nothing else in
the library names an architecture.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Mapping, Protocol

from .config.keys import ConfigError
from .config.spec import ModelSpec


class TypedConfig(Protocol):
    def model_spec(self) -> ModelSpec: ...
    def to_dict(self) -> dict[str, Any]: ...


@dataclass(frozen=True)
class Architecture:
    name: str
    parse: Callable[[Mapping[str, Any], Mapping[str, Any] | None], TypedConfig]


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, parse: Callable[..., TypedConfig], replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, parse)


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_of(config: Mapping[str, Any]) -> Architecture:
    archs = config.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("missing config key: architectures (a list with the model class name)")
    if archs[0] not in _ARCHITECTURES:
        raise ConfigError(f"unknown architecture {archs[0]!r}; known: {', '.join(known_architectures())}")
    return _ARCHITECTURES[archs[0]]


def parse_config(config: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> TypedConfig:
    return architecture_of(config).parse(config, generation)


def read_config_folder(folder: str) -> TypedConfig:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {folder}")
    with open(path) as f:
        try:
            config = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(config, dict):
        raise ConfigError(f"{path}: the top level is not an object")
    generation = None
    gpath = os.path.join(folder, "generation_config.json")
    if os.path.isfile(gpath):
        with open(gpath) as f:
            generation = json.load(f)
    return parse_config(config, generation)


def _register_builtin() -> None:
    from .config.qwen3 import ARCHITECTURE, Qwen3Config
    register_architecture(ARCHITECTURE, Qwen3Config.from_dict, replace=True)


_register_builtin()
