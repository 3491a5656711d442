"""Token embedding (row gather, no scaling) and the output head.

crates/llm-backend/src/core/qwen/ops/embedding.rs:26-36 (gather, error for an id outside
the vocabulary) and crates/llm-backend/src/core/qwen/ops/lm_head.rs:68-86 of the
reference; a tied head names the embedding table (crates/llm-models/src/qwen.rs:282-288),
and both then share one device buffer.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import Part, Runtime, WeightSpec


def _table(weights, rt: Runtime, name: str, hidden_size: int):
    """The table [V, H] on the device, one copy per stored tensor: in the tensor-core product's box layout
    where that kernel takes it (bfloat16, H a multiple of 8; the embedding gathers rows from the boxes), else
    row-major."""
    if rt.dtype == torch.bfloat16 and hidden_size % 8 == 0:
        def make():
            return rt.ops.tile_weight(weights.stored(name).to(device=rt.device, dtype=rt.dtype))
        return weights.shared((name, "boxes"), make)
    return weights.on_device(name, rt.dtype)


class Embedding(Part):
    capture_safe = True
    kernels_only = True

    def __init__(self, weight_name: str, vocab_size: int, hidden_size: int):
        self.weight_name, self.vocab_size, self.hidden_size = weight_name, vocab_size, hidden_size
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.vocab_size, self.hidden_size), "embedding")}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.table = _table(weights, rt, self.weight_name, self.hidden_size)

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        """The 32-bit residual stream [T, H] that the blocks add into."""
        return self.rt.ops.embedding(self.table, token_ids)


class OutputHead(Part):
    """Logits = W x in 32-bit, W [V, H] (its own tensor, or the embedding table when tied)."""

    capture_safe = True
    kernels_only = True

    def __init__(self, weight_name: str, vocab_size: int, hidden_size: int):
        self.weight_name, self.vocab_size, self.hidden_size = weight_name, vocab_size, hidden_size
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.vocab_size, self.hidden_size), "embedding")}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.weight = _table(weights, rt, self.weight_name, self.hidden_size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.rt.ops.linear(x, self.weight, torch.float32)
