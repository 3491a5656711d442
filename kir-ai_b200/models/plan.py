"""A model as data: parts, and the order in which the blocks run.

``ModelPlan`` holds an embedding, a list of blocks, the ``order`` (a list of
``LayerCall``), a final norm and an output head.  The order may name a block
twice (weights shared between depths; each call then has a cache of its own)
and a call may read the cache that an earlier call filled (``write`` false).
``DecoderModel`` runs a plan on a batch; it knows nothing of any architecture.

The reference hard-codes the loop over ``spec.num_hidden_layers``
(crates/llm-backend/src/core/qwen/ops/decoder.rs:481-515 prefill, :526-566 decode).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..parts.base import Norm, Runtime, WeightSpec
from ..parts.block import Block
from ..parts.embedding import Embedding, OutputHead


@dataclass(frozen=True)
class LayerCall:
    """Run ``block`` with cache layer ``cache`` (None: the mixer keeps nothing);
    ``write`` false reads what an earlier call wrote in the same step."""

    block: int
    cache: Optional[int] = None
    write: bool = True


class PlanError(ValueError):
    pass


@dataclass
class ModelPlan:
    embedding: Embedding
    blocks: List[Block]
    order: List[LayerCall]
    final_norm: Norm
    head: OutputHead
    vocab_size: int
    hidden_size: int
    max_positions: Optional[int] = None
    ignorable_weights: List[str] = field(default_factory=list)  # tensors a folder may hold that no part wants
    cache_needs: List[object] = field(default_factory=list)  # filled by validate(): one need per cache layer

    def validate(self) -> "ModelPlan":
        """Checks the order against the blocks and derives the need of every cache layer."""
        needs: Dict[int, object] = {}
        for step, call in enumerate(self.order):
            if not 0 <= call.block < len(self.blocks):
                raise PlanError(f"order[{step}] names block {call.block}, but there are {len(self.blocks)} blocks")
            need = self.blocks[call.block].mixer.cache_need()
            if need is None:
                if call.cache is not None:
                    raise PlanError(f"order[{step}]: block {call.block}'s mixer keeps nothing, yet cache {call.cache} is named")
                continue
            if call.cache is None:
                raise PlanError(f"order[{step}]: block {call.block}'s mixer needs a cache layer")
            if call.write:
                if call.cache in needs:
                    raise PlanError(f"order[{step}]: cache layer {call.cache} is written by two calls")
                needs[call.cache] = need
            else:
                if call.cache not in needs:
                    raise PlanError(f"order[{step}]: cache layer {call.cache} is read before any call wrote it")
                if needs[call.cache] != need:
                    raise PlanError(f"order[{step}]: reader needs {need}, cache layer {call.cache} holds {needs[call.cache]}")
        if sorted(needs) != list(range(len(needs))):
            raise PlanError(f"cache layers must be numbered 0..n-1 without gaps, got {sorted(needs)}")
        self.cache_needs = [needs[i] for i in range(len(needs))]
        return self

    def parts(self):
        return [self.embedding, *self.blocks, self.final_norm, self.head]

    def capture_safe(self) -> bool:
        """Whether a step of single tokens may be recorded into a CUDA graph: every part promises it
        (``Part.capture_safe``)."""
        return all(bool(getattr(part, "capture_safe", False)) for part in self.parts())

    def kernels_only(self) -> bool:
        """Whether products may be held back and launched together: every part promises to touch activations
        through the kernels only (``Part.kernels_only``)."""
        return all(bool(getattr(part, "kernels_only", False)) for part in self.parts())

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs: Dict[str, WeightSpec] = {}
        for part in self.parts():
            for name, spec in part.weight_specs().items():
                if name in specs and specs[name].shape != spec.shape:
                    raise PlanError(f"tensor {name} is wanted with shapes {specs[name].shape} and {spec.shape}")
                specs[name] = spec
        return specs


class DecoderModel:
    """Runs a plan: embedding, the blocks in ``order``, and logits at chosen rows."""

    def __init__(self, plan: ModelPlan, rt: Runtime):
        self.plan = plan.validate()
        self.rt = rt
        # with parts that touch activations through the kernels only, a step's small products are launched together
        self._kernels_only = plan.kernels_only() and hasattr(rt.ops, "chained_products")
        self.nvtx = False  # True: every layer call is an NVTX range (the reference counts attempts and fallbacks per
        # kernel instead, crates/llm-native-runtime/src/native_metrics.rs:7-70; here ops.launch_counts does that)

    def load(self, weights) -> "DecoderModel":
        for part in self.plan.parts():
            part.load(weights, self.rt)
        return self

    def forward(self, batch, cache) -> tuple:
        """The residual stream [T, H] (32-bit) and the last block's not-yet-added output."""
        nvtx = torch.cuda.nvtx if self.nvtx else None  # ranges around the layer calls, for a timeline tool
        with self.rt.ops.chained_products(self._kernels_only):
            resid = self.plan.embedding.forward(batch.token_ids)
            delta = None
            order = self.plan.order
            for i, call in enumerate(order):
                view = cache.layer_view(call.cache) if call.cache is not None else None
                following = self.plan.blocks[order[i + 1].block] if i + 1 < len(order) else None
                if nvtx:
                    nvtx.range_push(f"layer call {i}: block {call.block}, {batch.num_tokens} tokens")
                resid, delta = self.plan.blocks[call.block].forward(resid, delta, batch, view, call.write, following)
                if nvtx:
                    nvtx.range_pop()
        return resid, delta

    def logits(self, resid: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor) -> torch.Tensor:
        """32-bit logits [len(rows), V] of the token rows ``rows`` (int32, on the device)."""
        with self.rt.ops.chained_products(self._kernels_only):
            normed = self.plan.final_norm.add_forward_rows(resid, delta, rows)
            logits = self.plan.head.forward(normed)
        return logits
