"""A loaded model with its cache: what the step function, the scheduler, the
command line and trace replay all drive.

``ModelRunner.from_folder`` reads config.json, picks the architecture from the
registry, checks and loads the weights, and makes the cache pool.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..cache.manager import CacheManager
from ..models.plan import DecoderModel
from ..parts.base import Runtime
from ..registry import load_config, plan_for_config
from ..weights import loader as weight_loader
from ..weights.random_init import random_tensors
from .batch import StepEntry
from .step import run_step

_DTYPES = {"float32": torch.float32, "fp32": torch.float32, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    if name not in _DTYPES:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {name!r}")
    return _DTYPES[name]


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError(
            "kirai_b200 runs on a CUDA device (sm_100a) only; there is no CPU path "
            f"(asked for {device}, torch.cuda.is_available() = {torch.cuda.is_available()})"
        )
    return device


class ModelRunner:
    def __init__(self, config, model: DecoderModel, cache: CacheManager):
        self.config, self.model, self.cache = config, model, cache
        self.rt = model.rt

    @classmethod
    def build(cls, config, weights_source_factory, *, dtype="bfloat16", device="cuda:0", page_size: int = 16,
              max_tokens: Optional[int] = None, num_pages: Optional[int] = None, num_slots: int = 64) -> "ModelRunner":
        device = require_cuda(device)
        rt = Runtime(device, parse_dtype(dtype))
        rt.ops.library()  # builds or loads the kernels now; a missing library fails here, loudly
        plan = plan_for_config(config)
        model = DecoderModel(plan, rt)
        source = weights_source_factory(plan.weight_specs(), device, plan.ignorable_weights)
        model.load(source)
        source.forget()
        cache = CacheManager(plan.cache_needs, page_size=page_size, num_slots=num_slots, dtype=rt.dtype, device=device,
                             num_pages=num_pages, max_tokens=max_tokens)
        return cls(config, model, cache)

    @classmethod
    def from_folder(cls, model_dir: str, **kwargs) -> "ModelRunner":
        config = load_config(model_dir)
        return cls.build(config, lambda specs, device, ignorable: weight_loader.open_checked(model_dir, specs, device, ignorable), **kwargs)

    @classmethod
    def from_random(cls, config, seed: int, *, std: float = 0.02, norm_jitter: float = 0.0, **kwargs) -> "ModelRunner":
        """Random weights made on the device, without a model folder (for measurements at real sizes)."""
        def factory(specs, device, ignorable):
            tensors = random_tensors(specs, seed, std=std, norm_jitter=norm_jitter, dtype=torch.bfloat16, device=device)
            return weight_loader.from_tensors(tensors, specs, device, ignorable)
        return cls.build(config, factory, **kwargs)

    def step(self, entries: Sequence[StepEntry], **kwargs):
        return run_step(self.model, self.cache, entries, **kwargs)
