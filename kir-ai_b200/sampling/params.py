"""Sampling options of a request, with the reference's names, defaults and ranges.

``temperature`` 0 is greedy, else nucleus sampling with ``top_p`` (1.0 keeps the
whole vocabulary); defaults 1.0 and 1.0; temperature finite in [0, 2], top_p
finite in (0, 1] (crates/llm-util/src/sampling.rs:3-5,34-49,
crates/llm-backend-contracts/src/lib.rs:548-598).  ``max_new_tokens`` is the
request's ``max_tokens`` (crates/llm-native-runtime/src/native_text/generation.rs:17-33).
The reference seeds its generator from the system and offers no seed; ``seed``
here makes a run repeatable.  ``eos_token_id`` stands in for the reference's stop
token looked up in the tokenizer (crates/llm-native-runtime/src/native_qwen.rs:277-283).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    seed: Optional[int] = None
    max_new_tokens: Optional[int] = None  # None: the engine's default (--max-new-tokens)
    eos_token_id: Optional[int] = None
    ignore_eos: bool = False

    def __post_init__(self):
        if not math.isfinite(self.temperature) or not 0.0 <= self.temperature <= 2.0:
            raise ValueError(f"temperature must be finite and within [0, 2], got {self.temperature}")
        if not math.isfinite(self.top_p) or not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must be finite and within (0, 1], got {self.top_p}")
        if self.max_new_tokens is not None and self.max_new_tokens < 1:
            raise ValueError("max_tokens must be greater than 0")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0
