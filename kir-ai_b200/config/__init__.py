"""Typed configurations, one class per architecture, read from config.json."""
from .base import ConfigError, read_config_json
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "read_config_json", "Qwen3Config"]
