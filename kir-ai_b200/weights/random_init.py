"""Random weights from a configuration and a seed.

``random_tensors`` fills every tensor that a model's parts declare, by role:
linear matrices and embeddings from N(0, std), norm weights from
1 + N(0, norm_jitter) (jitter 0 gives ones), integer tables uniformly.
``write_random_model`` writes a model folder (config.json, model.safetensors).
Tensors are generated one by one from a generator seeded with (seed, name), so
a tensor's values do not depend on which other tensors exist or on the device
that will hold them.

The reference has no such mode; its tests hand-write tiny tensors
(crates/llm-native-runtime/src/native_qwen/tests/fixtures.rs:70-135).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Mapping

import torch

from ..parts.base import WeightSpec
from .safetensors_io import write_safetensors


def _generator(seed: int, name: str, device="cpu") -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    generator = torch.Generator(device=device)
    generator.manual_seed(int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF)
    return generator


def random_tensors(specs: Mapping[str, WeightSpec], seed: int, *, std: float = 0.02, norm_jitter: float = 0.1,
                   dtype: torch.dtype = torch.bfloat16, device="cpu", int_table_range: int = 16) -> Dict[str, torch.Tensor]:
    tensors: Dict[str, torch.Tensor] = {}
    for name, spec in specs.items():
        generator = _generator(seed, name, device)
        if spec.role == "int_table":
            tensors[name] = torch.randint(0, int_table_range, spec.shape, generator=generator, device=device, dtype=torch.int32)
            continue
        values = torch.randn(spec.shape, generator=generator, device=device, dtype=torch.float32)
        if spec.role == "norm":
            values = 1.0 + norm_jitter * values
        else:
            values = std * values
        tensors[name] = values.to(dtype)
    return tensors


def write_random_model(model_dir: str, config, seed: int, *, std: float = 0.02, norm_jitter: float = 0.1,
                       dtype: torch.dtype = torch.bfloat16) -> None:
    """Writes ``config.json`` and ``model.safetensors`` for ``config`` (a typed configuration
    of a registered architecture) with random weights."""
    from ..registry import plan_for_config

    plan = plan_for_config(config)
    tensors = random_tensors(plan.weight_specs(), seed, std=std, norm_jitter=norm_jitter, dtype=dtype)
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(config.to_dict(), handle, indent=2)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors, metadata={"format": "pt", "seed": str(seed)})
