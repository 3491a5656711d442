"""Dense SwiGLU feed-forward: down(silu(gate x) * (up x)), silu(x) = x / (1 + e^-x).

crates/llm-backend/src/core/qwen/ops/moe.rs:31-88 and
crates/llm-backend/src/core/math.rs:196-225 of the reference.  No biases.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import FeedForward, Runtime, WeightSpec
from .linear import Linear


class SwiGLU(FeedForward):
    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, names: Optional[Dict[str, str]] = None):
        n = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        n.update(names or {})
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.gate_up = Linear([(prefix + n["gate"], intermediate_size), (prefix + n["up"], intermediate_size)], hidden_size)
        self.down = Linear([(prefix + n["down"], hidden_size)], intermediate_size)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {**self.gate_up.weight_specs(), **self.down.weight_specs()}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.gate_up.load(weights, rt)
        self.down.load(weights, rt)

    def forward(self, x: torch.Tensor, batch=None) -> torch.Tensor:
        gate_up = self.gate_up.forward(x)
        return self.down.forward(self.rt.ops.swiglu(gate_up))
