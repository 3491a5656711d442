"""A bias-free linear layer over one or several stored matrices.

The matrices named in ``sources`` ([out_i, in] each, row-major as stored) are
stacked along the output axis at load, so that projections that read the same
input (q, k, v; gate, up) run as one product.  The reference keeps them apart
and reads them under their stored names
(crates/llm-backend/src/core/qwen/ops/attention_full.rs:586-609).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .base import Part, Runtime, WeightSpec


class Linear(Part):
    def __init__(self, sources: Sequence[Tuple[str, int]], in_features: int):
        self.sources: List[Tuple[str, int]] = list(sources)
        self.in_features = in_features
        self.out_features = sum(n for _, n in self.sources)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {name: WeightSpec((n, self.in_features), "linear") for name, n in self.sources}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        if len(self.sources) == 1:
            self.weight = weights.on_device(self.sources[0][0], rt.dtype)
        else:
            parts = [weights.stored(name).to(device=rt.device, dtype=rt.dtype) for name, _ in self.sources]
            self.weight = torch.cat(parts, dim=0).contiguous()

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return self.rt.ops.linear(x, self.weight, out_dtype)
