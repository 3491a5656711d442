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

    # Largest batch for which a norm is folded into the products around it: every batch that the weight-streaming
    # products take.  Measured on the 8B layer sizes (ms a decode step, folded against separate): one request 4 %
    # faster, 24 requests of 2,048 tokens 4.42, 32 requests 4.70 against 4.83, 48 of 1,024 tokens 4.84 against 4.97,
    # 64 of 4,096 tokens 9.51 against 9.54.  (Before the epilogue stored through shared memory it took 2.4 to 3.8 us a
    # product and lost from 17 rows on.)  The many-token kernel's epilogue of this kind is slower than the separate
    # norm kernel, beside which the next product already loads its first weight tiles.
    FUSED_NORM_MAX_ROWS = 64

    def on_tensor_cores(self) -> bool:
        """Whether this layer's products run on the tensor-core kernel, which alone has the fused epilogues."""
        return self.rt.dtype == torch.bfloat16 and self.in_features % 8 == 0

    def fuses_norms(self, rows: int) -> bool:
        """Whether a batch of ``rows`` tokens should have the norms next to this product folded into it."""
        return self.on_tensor_cores() and rows <= self.FUSED_NORM_MAX_ROWS

    def forward_into_norm(self, x: torch.Tensor, resid: torch.Tensor, spec: FusedNormSpec) -> UnscaledNorm:
        """resid += x W^T in place; returns the sum's rows under the norm ``spec`` without their 1 / rms factor."""
        rows, sumsq = self.rt.ops.linear_residual_norm(x, self.weight, resid, spec.weight)
        return UnscaledNorm(rows, sumsq, spec.width, spec.eps)
