"""Validation helpers shared by the config groups (reference: llmtuner/config/utils.py:1-77)."""
from __future__ import annotations

import dataclasses
from typing import Any

from ..errors import ConfigError


def require_integer_at_least(name: str, value: Any, minimum: int) -> int:
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(f"{name} must be an integer, got {value!r}")
    if value < minimum:
        raise ConfigError(f"{name} must be >= {minimum}, got {value}")
    return value


def require_bool(name: str, value: Any) -> bool:
    if not isinstance(value, bool):
        raise ConfigError(f"{name} must be a bool, got {value!r}")
    return value


def require_choice(name: str, value: Any, choices) -> Any:
    if value not in choices:
        raise ConfigError(f"{name} must be one of {sorted(map(str, choices))}, got {value!r}")
    return value


def require_string_patterns(name: str, value: Any) -> list[str]:
    if not isinstance(value, (list, tuple)) or not all(isinstance(v, str) and v for v in value):
        raise ConfigError(f"{name} must be a list of non-empty strings, got {value!r}")
    return list(value)


def rebuild_config_group(cls: type, source: Any, **overrides: Any):
    """A fresh instance of `cls` from a dict or another instance, so `__post_init__` re-validates."""
    if source is None:
        data = {}
    elif dataclasses.is_dataclass(source):
        data = {f.name: getattr(source, f.name) for f in dataclasses.fields(source) if f.init}
    else:
        data = dict(source)
    data.update(overrides)
    names = {f.name for f in dataclasses.fields(cls) if f.init}
    unknown = set(data) - names
    if unknown:
        raise ConfigError(f"{cls.__name__}: unknown fields {sorted(unknown)}")
    return cls(**data)
