"""Typed readers for config.json keys.

Every structural key is required; a missing key is an error that names the key
and nothing is guessed, following the reference's loader
(mynah-slm src/model.c:11-13, :41-69). The float reader accepts a JSON integer
(`"rope_theta": 1000000`) and the integer reader refuses a float, the JSON
twin of the reference's float-read-as-integer trap (src/model.c:61-64).
"""
from __future__ import annotations

from typing import Any, Mapping


class ConfigError(ValueError):
    """A config.json that this library cannot or will not run."""


_MISSING = object()


def _get(d: Mapping[str, Any], key: str, default: Any = _MISSING) -> Any:
    if key not in d or d[key] is None and default is not _MISSING:
        if default is _MISSING:
            raise ConfigError(f"missing config key: {key}")
        return default
    return d[key]


def req_int(d: Mapping[str, Any], key: str, minimum: int | None = 1) -> int:
    v = _get(d, key)
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"{key} is not an integer: {v!r}")
    if minimum is not None and v < minimum:
        raise ConfigError(f"{key} must be >= {minimum}, got {v}")
    return v


def opt_int(d: Mapping[str, Any], key: str, default: int | None) -> int | None:
    v = _get(d, key, default)
    if v is None:
        return None
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"{key} is not an integer: {v!r}")
    return v


def req_float(d: Mapping[str, Any], key: str) -> float:
    v = _get(d, key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"{key} is not a float: {v!r}")
    return float(v)


def req_bool(d: Mapping[str, Any], key: str) -> bool:
    v = _get(d, key)
    if not isinstance(v, bool):
        raise ConfigError(f"{key} is not a boolean: {v!r}")
    return v


def opt_bool(d: Mapping[str, Any], key: str, default: bool) -> bool:
    v = _get(d, key, default)
    if not isinstance(v, bool):
        raise ConfigError(f"{key} is not a boolean: {v!r}")
    return v


def req_str(d: Mapping[str, Any], key: str) -> str:
    v = _get(d, key)
    if not isinstance(v, str):
        raise ConfigError(f"{key} is not a string: {v!r}")
    return v


def int_set(v: Any, key: str) -> tuple[int, ...]:
    """An id or a list of ids (`eos_token_id` comes in both forms)."""
    if v is None:
        return ()
    if isinstance(v, int) and not isinstance(v, bool):
        return (v,)
    if isinstance(v, (list, tuple)) and all(isinstance(x, int) and not isinstance(x, bool) for x in v):
        return tuple(v)
    raise ConfigError(f"{key} is neither an integer nor a list of integers: {v!r}")
