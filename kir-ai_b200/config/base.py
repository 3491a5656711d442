"""Helpers shared by every architecture's typed configuration.

A configuration class reads the architecture's own ``config.json`` keys and
nothing else: no size and no constant that ``config.json`` gives is written in
code.  Errors carry a stable ``code`` in the manner of the reference's
``ModelSpecError`` (crates/llm-models/src/qwen.rs:445-471): a missing or
unsupported option is ``unsupported_capability``, a malformed value is
``invalid_request``.
"""
from __future__ import annotations

import json
import os
from typing import Any, Mapping


class ConfigError(ValueError):
    """A config.json that this framework cannot run; ``code`` names the kind."""

    def __init__(self, code: str, message: str):
        super().__init__(f"{code}: {message}")
        self.code = code
        self.message = message

    @classmethod
    def unsupported(cls, message: str) -> "ConfigError":
        return cls("unsupported_capability", message)

    @classmethod
    def invalid(cls, message: str) -> "ConfigError":
        return cls("invalid_request", message)


def read_config_json(model_dir: str | os.PathLike) -> dict:
    """Reads ``config.json`` of a model folder into a dict."""
    path = os.path.join(os.fspath(model_dir), "config.json")
    try:
        with open(path, "r", encoding="utf-8") as handle:
            raw = json.load(handle)
    except FileNotFoundError:
        raise ConfigError("model_artifact_missing", f"no config.json in {model_dir}") from None
    except json.JSONDecodeError as err:
        raise ConfigError.invalid(f"invalid JSON: {err}") from None
    if not isinstance(raw, dict):
        raise ConfigError.invalid("config.json must hold a JSON object")
    return raw


def required_int(raw: Mapping[str, Any], key: str, family: str, *, minimum: int = 1) -> int:
    value = raw.get(key)
    if value is None:
        raise ConfigError.unsupported(f"{family} config missing {key}")
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError.invalid(f"{family} config {key} must be an integer, got {value!r}")
    if value < minimum:
        raise ConfigError.invalid(f"{family} config {key} must be >= {minimum}, got {value}")
    return value


def required_float(raw: Mapping[str, Any], key: str, family: str) -> float:
    value = raw.get(key)
    if value is None:
        raise ConfigError.unsupported(f"{family} config missing {key}")
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError.invalid(f"{family} config {key} must be a number, got {value!r}")
    return float(value)


def optional_int(raw: Mapping[str, Any], key: str, family: str, default, *, minimum: int = 0):
    value = raw.get(key)
    if value is None:
        return default
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError.invalid(f"{family} config {key} must be an integer, got {value!r}")
    if value < minimum:
        raise ConfigError.invalid(f"{family} config {key} must be >= {minimum}, got {value}")
    return value


def optional_bool(raw: Mapping[str, Any], key: str, family: str, default: bool) -> bool:
    value = raw.get(key)
    if value is None:
        return default
    if not isinstance(value, bool):
        raise ConfigError.invalid(f"{family} config {key} must be true or false, got {value!r}")
    return value
