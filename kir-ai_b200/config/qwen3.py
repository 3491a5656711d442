"""Typed configuration of the Qwen3 dense decoder (``Qwen3ForCausalLM``).

Keys, defaults and refusals follow the reference's ``QwenModelSpec``
(crates/llm-models/src/qwen.rs:163-213 fields, :349-368 unsupported options,
:370-385 sliding window, :387-408 the keys that are read).  One addition:
``max_window_layers``.  The reference does not read it and applies an enabled
window to every layer (crates/llm-backend/src/core/qwen/ops/cache.rs:116-121);
here layer ``i`` is windowed when ``use_sliding_window`` and
``i >= max_window_layers``, and the default ``0`` reproduces the reference.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any, Mapping, Optional

from .base import (
    ConfigError,
    optional_bool,
    optional_int,
    required_float,
    required_int,
)

_FAMILY = "qwen"


@dataclass(frozen=True)
class Qwen3Config:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: int = 0

    architecture = "Qwen3ForCausalLM"
    model_type = "qwen3"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Qwen3Config":
        architectures = raw.get("architectures") or []
        if not architectures:
            raise ConfigError.unsupported("model config missing architecture")
        if architectures[0] != cls.architecture or raw.get("model_type") != cls.model_type:
            raise ConfigError.unsupported(
                f"config is not a Qwen3 dense architecture: architectures[0]={architectures[0]!r}, "
                f"model_type={raw.get('model_type')!r}"
            )
        hidden_act = raw.get("hidden_act")
        if hidden_act is not None and hidden_act != "silu":
            raise ConfigError.unsupported(
                f"qwen3 dense hidden_act `{hidden_act}` is unsupported; only `silu` is supported"
            )
        if raw.get("attention_bias") not in (None, False):
            raise ConfigError.unsupported("qwen3 dense attention_bias=true is unsupported")
        if raw.get("rope_scaling") is not None:
            raise ConfigError.unsupported("qwen3 dense rope_scaling is unsupported")

        hidden_size = required_int(raw, "hidden_size", _FAMILY)
        heads = required_int(raw, "num_attention_heads", _FAMILY)
        kv_heads = required_int(raw, "num_key_value_heads", _FAMILY)
        head_dim = optional_int(raw, "head_dim", _FAMILY, None, minimum=1)
        if head_dim is None:
            head_dim = hidden_size // heads
        if heads % kv_heads != 0:
            raise ConfigError.invalid(
                f"qwen config num_attention_heads {heads} is not a multiple of "
                f"num_key_value_heads {kv_heads}"
            )
        if head_dim % 2 != 0:
            raise ConfigError.invalid(f"qwen config head_dim {head_dim} must be even for rotary pairs")

        use_window = optional_bool(raw, "use_sliding_window", _FAMILY, False)
        window = None
        if use_window:
            window = raw.get("sliding_window")
            if window is None:
                raise ConfigError.invalid("qwen3 dense use_sliding_window=true requires sliding_window")
            if isinstance(window, bool) or not isinstance(window, int):
                raise ConfigError.invalid(f"qwen3 dense sliding_window must be an integer, got {window!r}")
            if window <= 0:
                raise ConfigError.invalid("qwen3 dense sliding_window must be greater than 0")
        eps = required_float(raw, "rms_norm_eps", _FAMILY)
        if eps < 0.0:
            raise ConfigError.invalid("qwen config rms_norm_eps must be non-negative")
        return cls(
            hidden_size=hidden_size,
            intermediate_size=required_int(raw, "intermediate_size", _FAMILY),
            num_hidden_layers=required_int(raw, "num_hidden_layers", _FAMILY),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=required_int(raw, "vocab_size", _FAMILY),
            max_position_embeddings=required_int(raw, "max_position_embeddings", _FAMILY),
            rms_norm_eps=eps,
            rope_theta=required_float(raw, "rope_theta", _FAMILY),
            tie_word_embeddings=optional_bool(raw, "tie_word_embeddings", _FAMILY, False),
            use_sliding_window=use_window,
            sliding_window=window,
            max_window_layers=optional_int(raw, "max_window_layers", _FAMILY, 0) if use_window else 0,
        )

    def window_for_layer(self, layer: int) -> Optional[int]:
        """Window width of ``layer``, or None when it sees every earlier token."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return None

    def to_dict(self) -> dict:
        """The config.json content that parses back to this configuration."""
        out = asdict(self)
        out["architectures"] = [self.architecture]
        out["model_type"] = self.model_type
        out["hidden_act"] = "silu"
        out["attention_bias"] = False
        out["rope_scaling"] = None
        if not self.use_sliding_window:
            out.pop("sliding_window")
            out.pop("max_window_layers")
        return out
