"""Dense SwiGLU feed-forward: down(silu(gate x) * (up x)), silu(x) = x / (1 + e^-x).

crates/llm-backend/src/core/qwen/ops/moe.rs:31-88 and
crates/llm-backend/src/core/math.rs:196-225 of the reference.  No biases.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import FeedForward, Runtime, UnscaledNorm, WeightSpec
from .linear import Linear


class SwiGLU(FeedForward):
    capture_safe = True
    kernels_only = True

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
        self.down.load(weights, rt)
        # On the tensor cores gate and up are one product whose epilogue applies silu(gate) * up:
        # their rows are interleaved in eights at load, so that a thread's 16 outputs pair up.
        self.fused_weight = None
        if rt.dtype == torch.bfloat16 and self.intermediate_size % 8 == 0 and self.hidden_size % 8 == 0:
            (gate_name, _), (up_name, _) = self.gate_up.sources
            gate = weights.stored(gate_name).to(device=rt.device, dtype=rt.dtype)
            up = weights.stored(up_name).to(device=rt.device, dtype=rt.dtype)
            self.fused_weight = rt.ops.tile_weight(rt.ops.interleave_gate_up(gate, up))
        else:
            self.gate_up.load(weights, rt)

    def takes_unscaled(self, rows: int) -> bool:
        return self.fused_weight is not None and self.down.fuses_norms(rows)

    def fuses_into_norm(self, rows: int) -> bool:
        return self.fused_weight is not None and self.down.fuses_norms(rows)

    def forward(self, x, batch=None) -> torch.Tensor:
        return self.down.forward(self._activation(x))

    def forward_into_norm(self, x, batch, resid, spec):
        return self.down.forward_into_norm(self._activation(x), resid, spec)

    def _activation(self, x) -> torch.Tensor:
        """silu(gate x) * (up x): [T, I]."""
        ops = self.rt.ops
        if isinstance(x, UnscaledNorm):
            return ops.linear_tcgen05(x.rows, self.fused_weight, swiglu=True, row_scale=x.row_scale())
        if self.fused_weight is not None and ops.tcgen05_takes(x):
            return ops.linear_tcgen05(x, self.fused_weight, swiglu=True)
        if self.fused_weight is not None:
            raise ValueError("SwiGLU input is not laid out for the tensor-core kernel (rows must be 16-byte aligned)")
        return ops.swiglu(self.gate_up.forward(x))
