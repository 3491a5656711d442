"""Interfaces of the parts a model is put together from.

A model is an embedding, a list of blocks, an order in which the blocks run, a
final norm and an output head.  A block arranges two norms, a mixer (attention
here) and a feed-forward.  Every part takes its sizes and constants as
constructor arguments, names the tensors it wants in ``weight_specs`` and picks
them up in ``load``; no part knows which model it sits in.  ``forward`` methods
work on a flat batch of tokens described by a ``StepBatch``
(kirai_b200.engine.batch).

The reference reaches the same separation with functions that take a spec and
flags (crates/llm-backend/src/core/native_attention.rs:11-17,109-116 generic
attention dims, crates/llm-backend/src/core/qwen/ops/attention_full.rs:41-48
per-variant flags).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class WeightSpec:
    """Shape and role of one named tensor.  The role tells the random-weights
    mode how to fill it and the loader which dtype family it must have:
    ``linear`` and ``embedding`` are floating matrices, ``norm`` a floating
    vector, ``int_table`` an integer table (kept as int32)."""

    shape: Tuple[int, ...]
    role: str = "linear"


@dataclass(frozen=True)
class KVCacheNeed:
    """A mixer that keeps keys and values of earlier tokens in pages.
    ``window`` None keeps every token; a width W keeps the last W."""

    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """A mixer that keeps a fixed-size state per request in a slot."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class FusedNormSpec:
    """What a product needs to take over a norm: y = x / sqrt(mean(x^2) + eps) * weight over ``width`` columns."""

    weight: torch.Tensor  # [width], float32
    eps: float
    width: int


@dataclass
class UnscaledNorm:
    """Normed rows without their 1 / rms factor: ``rows`` = stream * weight in the runtime dtype, and the parts
    ``sumsq`` [P, T] (float32) of each row's sum of squares.  The product that reads the rows multiplies its result
    by 1 / sqrt(sum_p sumsq[p] / width + eps), which commutes with the product."""

    rows: torch.Tensor
    sumsq: torch.Tensor
    width: int
    eps: float

    def row_scale(self):
        return (self.sumsq, self.width, self.eps)


class Runtime:
    """Where and in which precision a model runs: the device, the dtype of
    weights and activations (``torch.float32`` for the true 32-bit path,
    ``torch.bfloat16`` for serving), and the kernel namespace ``ops``."""

    def __init__(self, device: torch.device | str, dtype: torch.dtype, ops=None):
        self.device = torch.device(device)
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"runtime dtype must be float32 or bfloat16, got {dtype}")
        self.dtype = dtype
        if ops is None:
            from ..csrc import ops as _ops

            ops = _ops
        self.ops = ops


class Part:
    """Base of every part: the tensors it wants, and how it takes them.

    ``capture_safe`` true is a part's promise that, for a step in which every request brings one token, its
    ``forward`` can be recorded once into a CUDA graph and replayed with other inputs: it launches on the current
    stream only, never waits for the device, and takes everything that changes from step to step (tokens,
    positions, lengths, slots, block tables) from the batch's device tensors, not from its host copies
    (``start_positions``, ``slot_ids``; a captured step has none, and reading them raises).  A mixer with state of
    its own must also advance that state exactly once per run of the step.  The engine replays captured decode
    steps only for a plan all of whose parts promise this; otherwise every step runs eagerly.  The default is
    false, so a part written without thinking of graphs is never captured."""

    capture_safe = False

    # ``kernels_only`` true is a part's promise that it reads and writes activations through the kernels of
    # ``rt.ops`` only: no torch arithmetic on them, no copy to the host.  ``ops`` may then hold products back and
    # launch several of them as one kernel (``ops.chained_products``): a tensor that a product returns is filled only
    # when the next kernel of another kind is launched.  The model runs its blocks that way only when every part
    # promises this; otherwise every product is launched when it is asked for.
    kernels_only = False

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {}

    def load(self, weights, rt: Runtime) -> None:  # weights: kirai_b200.weights.loader.WeightSource
        self.rt = rt


class Norm(Part):
    """Normalisation over the last axis.

    ``forward(x)`` returns the normed rows in the runtime dtype.
    ``add_forward(resid, delta)`` first adds ``delta`` (runtime dtype, may be None)
    into the 32-bit residual stream ``resid`` in place, then norms the sum.
    """

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def add_forward(self, resid: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        raise NotImplementedError

    def fused_spec(self) -> Optional[FusedNormSpec]:
        """Optional: what the product before this norm needs to take it over (see ``Block``); None keeps
        the norm a kernel of its own."""
        return None


class PositionEncoding(Part):
    """Puts positions into queries and keys.  ``apply`` rewrites ``q`` [T, nq, d]
    and ``k`` [T, nkv, d] (row-strided views allowed) in place for the absolute
    ``positions`` [T] (int32, on the device)."""

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        raise NotImplementedError


class Mixer(Part):
    """Mixes information between the tokens of a request.

    ``cache_need`` says what it keeps between steps (None, KVCacheNeed or
    StateNeed).  ``forward(x, batch, cache, write_cache)`` gets the normed
    hidden rows [T, H], the batch description and a view of its cache layer
    (kirai_b200.cache.manager.KVLayerView or StateLayerView); when
    ``write_cache`` is false it reads a cache that another layer filled in this
    step and must not write it.

    Optional, for a block that fuses norms into products: ``takes_unscaled(rows)`` true means that for a
    batch of ``rows`` tokens ``forward`` accepts an ``UnscaledNorm`` in place of ``x``;
    ``fuses_into_norm(rows)`` true means the mixer has
    ``forward_into_norm(x, batch, cache, write_cache, resid, spec)``, which adds its output into the
    32-bit stream ``resid`` in place and returns the ``UnscaledNorm`` of the sum under ``spec``.
    """

    def cache_need(self):
        return None

    def forward(self, x: torch.Tensor, batch, cache, write_cache: bool = True) -> torch.Tensor:
        raise NotImplementedError

    def takes_unscaled(self, rows: int) -> bool:
        return False

    def fuses_into_norm(self, rows: int) -> bool:
        return False


class FeedForward(Part):
    """Token-wise transformation: ``forward(x, batch)`` maps [T, H] to [T, H].

    Optional, as for a mixer: ``takes_unscaled(rows)`` and ``fuses_into_norm(rows)`` with
    ``forward_into_norm(x, batch, resid, spec)``."""

    def forward(self, x: torch.Tensor, batch) -> torch.Tensor:
        raise NotImplementedError

    def takes_unscaled(self, rows: int) -> bool:
        return False

    def fuses_into_norm(self, rows: int) -> bool:
        return False
