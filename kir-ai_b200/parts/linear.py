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

from .base import FusedNormSpec, Part, Runtime, UnscaledNorm, WeightSpec


class Linear(Part):
    capture_safe = True
    kernels_only = True

    def __init__(self, sources: Sequence[Tuple[str, int]], in_features: int):
        self.sources: List[Tuple[str, int]] = list(sources)
        self.in_features = in_features
        self.out_features = sum(n for _, n in self.sources)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {name: WeightSpec((n, self.in_features), "linear") for name, n in self.sources}

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        parts = [weights.stored(name).to(device=rt.device, dtype=rt.dtype) for name, _ in self.sources]
        stacked = parts[0].contiguous() if len(parts) == 1 else torch.cat(parts, dim=0)
        # the tensor-core product streams weights fastest from its own box layout (``ops.TiledWeight``)
        self.weight = rt.ops.tile_weight(stacked) if self.on_tensor_cores() else stacked

    def forward(self, x, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        if isinstance(x, UnscaledNorm):
            return self.rt.ops.linear_tcgen05(x.rows, self.weight, out_dtype, row_scale=x.row_scale())
        return self.rt.ops.linear(x, self.weight, out_dtype)

    # Largest batch for which a norm is folded into the products around it.  Measured on the 8B layer sizes:
    # a decode step of one request gains 4 %, batches of 8 to 32 gain nothing, and from 64 rows on the separate
    # norm kernel wins, because the product after it loads its first weight tiles while the norm runs.
    FUSED_NORM_MAX_ROWS = 16
    # Where products are held back and run as one persistent kernel, the separate norm would cut that kernel in
    # two, and the weight stream that a folded norm once delayed runs on regardless: every batch that the
    # weight-streaming products take (up to 64 rows) has its norms folded in.
    FUSED_NORM_MAX_ROWS_CHAINED = 64

    def on_tensor_cores(self) -> bool:
        """Whether this layer's products run on the tensor-core kernel, which alone has the fused epilogues."""
        return self.rt.dtype == torch.bfloat16 and self.in_features % 8 == 0

    def fuses_norms(self, rows: int) -> bool:
        """Whether a batch of ``rows`` tokens should have the norms next to this product folded into it."""
        chaining = getattr(self.rt.ops, "chaining", None)
        limit = self.FUSED_NORM_MAX_ROWS_CHAINED if chaining is not None and chaining() else self.FUSED_NORM_MAX_ROWS
        return self.on_tensor_cores() and rows <= limit

    def forward_into_norm(self, x: torch.Tensor, resid: torch.Tensor, spec: FusedNormSpec) -> UnscaledNorm:
        """resid += x W^T in place; returns the sum's rows under the norm ``spec`` without their 1 / rms factor."""
        rows, sumsq = self.rt.ops.linear_residual_norm(x, self.weight, resid, spec.weight)
        return UnscaledNorm(rows, sumsq, spec.width, spec.eps)
