"""A block: two norms, a mixer and a feed-forward, and how they are arranged.

The residual stream is 32-bit; what a sub-layer produces (``delta``, in the
runtime dtype) is added into it by the next norm, so that sum and norm are one
pass over the row.  ``pre_norm`` is the reference's order
(crates/llm-backend/src/core/qwen/ops/decoder.rs:210-314): n1 = norm1(h);
a = mixer(n1); n2 = norm2(h + a); m = ffn(n2); out = h + a + m.  ``parallel``
feeds one norm to both sub-layers: out = h + mixer(n) + ffn(n).

Where the parts on both sides offer it, a norm is not a kernel of its own: the product before it adds into the
stream and writes the norm's rows without their 1 / rms factor (``forward_into_norm``), and the product after it
applies that factor to its result (``takes_unscaled``); see ``UnscaledNorm``.  The block asks the parts and falls
back to the separate norm kernel when either side declines, so a part without these methods still fits.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .base import FeedForward, FusedNormSpec, Mixer, Norm, Part, Runtime, UnscaledNorm, WeightSpec

ARRANGEMENTS = ("pre_norm", "parallel")


def _offers(part, method: str, rows: int) -> bool:
    """Whether a part has the optional ``method`` and answers yes for a batch of ``rows`` tokens; a part
    written without it declines."""
    fn = getattr(part, method, None)
    return bool(fn is not None and fn(rows))


class Block(Part):
    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Optional[Norm], ffn: FeedForward, arrangement: str = "pre_norm"):
        if arrangement not in ARRANGEMENTS:
            raise ValueError(f"unknown block arrangement {arrangement!r}; known: {ARRANGEMENTS}")
        if arrangement == "pre_norm" and norm2 is None:
            raise ValueError("the pre_norm arrangement needs a second norm")
        self.norm1, self.mixer, self.norm2, self.ffn, self.arrangement = norm1, mixer, norm2, ffn, arrangement

    def _parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.ffn) if p is not None]

    @property
    def capture_safe(self) -> bool:
        return all(bool(getattr(part, "capture_safe", False)) for part in self._parts())

    @property
    def kernels_only(self) -> bool:
        return all(bool(getattr(part, "kernels_only", False)) for part in self._parts())

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs: Dict[str, WeightSpec] = {}
        for part in self._parts():
            specs.update(part.weight_specs())
        return specs

    def load(self, weights, rt: Runtime) -> None:
        self.rt = rt
        for part in self._parts():
            part.load(weights, rt)

    def entry_spec(self, rows: int) -> Optional[FusedNormSpec]:
        """What the block before needs to take over this block's first norm for a batch of ``rows`` tokens;
        None if the norm stays a kernel."""
        if self.arrangement != "pre_norm" or not _offers(self.mixer, "takes_unscaled", rows):
            return None
        return self._spec(self.norm1)

    @staticmethod
    def _spec(norm) -> Optional[FusedNormSpec]:
        fn = getattr(norm, "fused_spec", None)
        return fn() if fn is not None else None

    def forward(self, resid: torch.Tensor, delta, batch, cache, write_cache: bool = True,
                following: Optional["Block"] = None) -> Tuple[torch.Tensor, object]:
        """Takes the stream and what the block before left: its not-yet-added output, or (if this block's
        ``entry_spec`` was offered to it as ``following``) the ``UnscaledNorm`` of the first norm.  Returns the
        stream and what this block leaves, in the same two forms."""
        rows = resid.shape[0]
        if self.arrangement == "pre_norm":
            n1 = delta if isinstance(delta, UnscaledNorm) else self.norm1.add_forward(resid, delta)
            spec2 = self._spec(self.norm2) if _offers(self.mixer, "fuses_into_norm", rows) and _offers(self.ffn, "takes_unscaled", rows) else None
            if spec2 is not None:
                n2 = self.mixer.forward_into_norm(n1, batch, cache, write_cache, resid, spec2)
            else:
                n2 = self.norm2.add_forward(resid, self.mixer.forward(n1, batch, cache, write_cache))
            spec_next = following.entry_spec(rows) if following is not None and _offers(self.ffn, "fuses_into_norm", rows) else None
            if spec_next is not None:
                return resid, self.ffn.forward_into_norm(n2, batch, resid, spec_next)
            return resid, self.ffn.forward(n2, batch)
        n = self.norm1.add_forward(resid, delta)
        a = self.mixer.forward(n, batch, cache, write_cache)
        m = self.ffn.forward(n, batch)
        self.norm1.rt.ops.add_into_residual(resid, a)
        return resid, m
