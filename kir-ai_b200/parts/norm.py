"""RMSNorm with the residual add fused in.

y = x * 1/sqrt(mean(x^2) + eps) * w, statistics in 32-bit, the scale 0 when
mean + eps is 0 (crates/llm-backend/src/core/math.rs:73-113 of the reference; the
dense model uses the plain weight, crates/llm-backend/src/core/qwen/ops/norm.rs:119-133).
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

from .base import FusedNormSpec, Norm, Runtime, WeightSpec


class RMSNorm(Norm):
    capture_safe = True
    kernels_only = True

    def __init__(self, weight_name: str, width: int, eps: float):
        self.weight_name = weight_name
        self.width = width
        self.eps = float(eps)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.width,), "norm")}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.weight = weights.on_device(self.weight_name, torch.float32)

    def add_forward(self, resid: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        return self.rt.ops.add_rmsnorm(resid, delta, self.weight, self.eps, self.rt.dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.rt.ops.add_rmsnorm(x, None, self.weight, self.eps, self.rt.dtype)

    def fused_spec(self) -> Optional[FusedNormSpec]:
        # the tensor-core products read and write rows in 16-byte units; KIRAI_FUSE_NORMS=0 keeps every norm a
        # kernel of its own (for comparing the two paths)
        if self.rt.dtype != torch.bfloat16 or self.width % 8 or os.environ.get("KIRAI_FUSE_NORMS", "1") == "0":
            return None
        return FusedNormSpec(self.weight, self.eps, self.width)

    def add_forward_rows(self, resid: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor) -> torch.Tensor:
        """The norm of ``resid[rows] + delta[rows]`` only; the stream is left untouched."""
        out, _ = self.rt.ops.add_rmsnorm(resid, delta, self.weight, self.eps, self.rt.dtype, row_index=rows)
        return out
