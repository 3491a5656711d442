"""A block: two norms, a mixer and a feed-forward, and how they are arranged.

The residual stream is 32-bit; what a sub-layer produces (``delta``, in the
runtime dtype) is added into it by the next norm, so that sum and norm are one
pass over the row.  ``pre_norm`` is the reference's order
(crates/llm-backend/src/core/qwen/ops/decoder.rs:210-314): n1 = norm1(h);
a = mixer(n1); n2 = norm2(h + a); m = ffn(n2); out = h + a + m.  ``parallel``
feeds one norm to both sub-layers: out = h + mixer(n) + ffn(n).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .base import FeedForward, Mixer, Norm, Part, Runtime, WeightSpec

ARRANGEMENTS = ("pre_norm", "parallel")


class Block(Part):
    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Optional[Norm], ffn: FeedForward, arrangement: str = "pre_norm"):
        if arrangement not in ARRANGEMENTS:
            raise ValueError(f"unknown block arrangement {arrangement!r}; known: {ARRANGEMENTS}")
        if arrangement == "pre_norm" and norm2 is None:
            raise ValueError("the pre_norm arrangement needs a second norm")
        self.norm1, self.mixer, self.norm2, self.ffn, self.arrangement = norm1, mixer, norm2, ffn, arrangement

    def _parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.ffn) if p is not None]

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs: Dict[str, WeightSpec] = {}
        for part in self._parts():
            specs.update(part.weight_specs())
        return specs

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        for part in self._parts():
            part.load(weights, rt)

    def forward(self, resid: torch.Tensor, delta: Optional[torch.Tensor], batch, cache, write_cache: bool = True
                ) -> Tuple[torch.Tensor, torch.Tensor]:
        """Takes the stream and the not-yet-added output of the block before;
        returns the stream and this block's not-yet-added output."""
        if self.arrangement == "pre_norm":
            n1 = self.norm1.add_forward(resid, delta)
            a = self.mixer.forward(n1, batch, cache, write_cache)
            n2 = self.norm2.add_forward(resid, a)
            return resid, self.ffn.forward(n2, batch)
        n = self.norm1.add_forward(resid, delta)
        a = self.mixer.forward(n, batch, cache, write_cache)
        m = self.ffn.forward(n, batch)
        self.norm1.rt.ops.add_into_residual(resid, a)
        return resid, m
