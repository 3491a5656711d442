"""Rotary position embedding, half-split pairing.

For i < rotary_dim/2: f_i = theta^(-2i/rotary_dim), angle = position * f_i (both
32-bit), and the pair (x_i, x_{i + rotary_dim/2}) is rotated by the angle
(crates/llm-backend/src/core/math.rs:515-529 of the reference).  The frequency
table is made once on the host in 32-bit and kept on the device.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import PositionEncoding, Runtime


class RotaryEmbedding(PositionEncoding):
    capture_safe = True
    kernels_only = True

    def __init__(self, head_dim: int, theta: float, rotary_dim: Optional[int] = None):
        self.head_dim = head_dim
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {head_dim}")
        self.theta = float(theta)
        self.inv_freq: Optional[torch.Tensor] = None

    def frequencies(self) -> torch.Tensor:
        half = self.rotary_dim // 2
        exponent = -(2.0 * torch.arange(half, dtype=torch.float32)) / float(self.rotary_dim)
        return torch.pow(torch.tensor(self.theta, dtype=torch.float32), exponent)

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        self.inv_freq = self.frequencies().to(rt.device)

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        self.rt.ops.rope_(q, positions, self.inv_freq, self.rotary_dim)
        self.rt.ops.rope_(k, positions, self.inv_freq, self.rotary_dim)

    def fused_table(self) -> Optional[torch.Tensor]:
        """The frequency table when the whole head is rotated (what the fused
        norm + rotation + cache-write kernel takes), else None."""
        return self.inv_freq if self.rotary_dim == self.head_dim else None
