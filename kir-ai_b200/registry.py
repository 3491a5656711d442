"""The one registry from an architecture's name to its configuration class and model.

``architectures[0]`` of config.json picks the entry.  An entry is a typed
configuration class (``from_dict``/``to_dict``) and a function that turns a
configuration into a ``ModelPlan``.  The reference dispatches on ``model_type``
with an enum (crates/llm-models/src/native_text.rs:55-68); here another
architecture is one ``register_architecture`` call.
"""
from __future__ import annotations

from typing import Callable, Dict, Tuple

from .config.base import ConfigError, read_config_json

_REGISTRY: Dict[str, Tuple[type, Callable]] = {}


def register_architecture(name: str, config_class: type, build_plan: Callable, *, replace: bool = False) -> None:
    if name in _REGISTRY and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _REGISTRY[name] = (config_class, build_plan)


def registered_architectures():
    return sorted(_REGISTRY)


def resolve(name: str) -> Tuple[type, Callable]:
    if name not in _REGISTRY:
        raise ConfigError.unsupported(
            f"architecture {name!r} is not registered; registered: {', '.join(registered_architectures()) or 'none'}"
        )
    return _REGISTRY[name]


def config_from_dict(raw: dict):
    architectures = raw.get("architectures") or []
    if not architectures:
        raise ConfigError.unsupported("model config missing architecture")
    config_class, _ = resolve(architectures[0])
    return config_class.from_dict(raw)


def load_config(model_dir: str):
    """The typed configuration of a model folder, its class chosen by config.json."""
    return config_from_dict(read_config_json(model_dir))


def plan_for_config(config):
    """The model plan of a typed configuration (the class carries its architecture name)."""
    _, build_plan = resolve(config.architecture)
    return build_plan(config)


def _register_builtin() -> None:
    from .config.qwen3 import Qwen3Config
    from .models.qwen3 import build_qwen3_plan

    register_architecture("Qwen3ForCausalLM", Qwen3Config, build_qwen3_plan, replace=True)


_register_builtin()
