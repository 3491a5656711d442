"""Helpers for tests that build parts and toy models directly: a runtime, weights from a
dict, and batches through the real cache manager and batch builder."""
from __future__ import annotations

import torch

import kirai_b200  # noqa: F401
from kirai_b200.cache import CacheManager
from kirai_b200.engine.batch import StepEntry, build_batch
from kirai_b200.parts.base import Runtime
from kirai_b200.weights.loader import from_tensors
from kirai_b200.weights.random_init import random_tensors

DEV = "cuda:0"


def runtime(dtype):
    return Runtime(DEV, dtype)


def load_part(part, dtype, seed=0, tensors=None):
    """Random weights for everything the part declares (or the given tensors); returns them on the CPU in 32-bit."""
    specs = part.weight_specs()
    tensors = tensors or random_tensors(specs, seed, std=0.08, norm_jitter=0.1, dtype=torch.bfloat16)
    part.load(from_tensors(tensors, specs, DEV), runtime(dtype))
    return {name: t.float() for name, t in tensors.items()}


class Session:
    """A cache manager and live requests, to make StepBatches the way the step function does."""

    def __init__(self, needs, dtype, page_size=4, num_pages=64, num_slots=4):
        self.cache = CacheManager(needs, page_size=page_size, num_pages=num_pages, num_slots=num_slots, dtype=dtype, device=DEV)
        self.requests = {}

    def batch(self, runs):
        """runs: list of (request name, tokens-or-count).  Reserves pages and builds the batch."""
        entries = []
        for name, tokens in runs:
            if name not in self.requests:
                self.requests[name] = self.cache.open(name)
            tokens = list(range(tokens)) if isinstance(tokens, int) else list(tokens)
            assert self.cache.reserve(self.requests[name], len(tokens))
            entries.append(StepEntry(self.requests[name], tokens, []))
        self._entries = entries
        return build_batch(entries, self.cache, DEV)

    def commit(self):
        for entry in self._entries:
            self.cache.commit(entry.request, len(entry.tokens))


def tolerance(dtype, reference):
    return 2e-5 * max(1.0, float(reference.abs().max())) if dtype == torch.float32 else 0.02 * float(reference.abs().max())
