"""The one step function.

``run_step`` takes a batch of (request, its next tokens, wanted places), in any
mix of prompt portions and single decoded tokens, runs exactly those tokens as
one batch from the cache that earlier steps left, writes their keys and values
to the requests' pages, and returns the 32-bit logits at the wanted places (in
the order of the entries and of ``want``).

The reference has two single-request entry points instead, a prefill chunk and
a decode step (crates/llm-native-runtime/src/native_qwen.rs:347-365,389-398), and runs
concurrent requests as independent threads.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .batch import StepEntry, build_batch


class OutOfPages(RuntimeError):
    """The step's tokens do not fit the free pages; nothing was taken."""


class StepError(ValueError):
    """A malformed step (bad token id, empty run, wanted place out of range...)."""


def check_entries(entries: Sequence[StepEntry], vocab_size: int, max_positions: Optional[int]) -> None:
    seen = set()
    for entry in entries:
        request = entry.request
        if id(request) in seen:
            raise StepError(f"request {request.request_id!r} appears twice in one step")
        seen.add(id(request))
        if request.closed:
            raise StepError(f"request {request.request_id!r} is closed")
        n = len(entry.tokens)
        if n == 0:
            raise StepError(f"request {request.request_id!r} brings no tokens")
        for token in entry.tokens:
            if not 0 <= int(token) < vocab_size:
                raise StepError(f"token id {token} outside vocab size {vocab_size}")
        for place in entry.want:
            if not 0 <= int(place) < n:
                raise StepError(f"request {request.request_id!r}: wanted place {place} is outside its {n} tokens")
        if max_positions is not None and request.length + n > max_positions:
            raise StepError(
                f"request {request.request_id!r}: {request.length + n} tokens exceed the model's {max_positions} positions"
            )


def reserve_all(entries: Sequence[StepEntry], cache) -> None:
    """Takes the pages for every entry, or none (OutOfPages)."""
    tables = cache.tables
    need = [0] * len(tables.pools)
    for entry in entries:
        for group, pages in enumerate(tables.pages_needed(entry.request, len(entry.tokens))):
            need[group] += pages
    for group, pool in enumerate(tables.pools):
        if need[group] > pool.free_pages:
            raise OutOfPages(f"cache group {group}: the step needs {need[group]} pages, {pool.free_pages} are free")
    for entry in entries:
        ok = cache.reserve(entry.request, len(entry.tokens))
        assert ok


def run_step(model, cache, entries: Sequence[StepEntry], *, check_errors: bool = True) -> Optional[torch.Tensor]:
    """Runs one step; returns logits [wanted, vocab] (float32, on the device) or None if nothing is wanted."""
    if not entries:
        return None
    check_entries(entries, model.plan.vocab_size, model.plan.max_positions)
    reserve_all(entries, cache)
    batch = build_batch(entries, cache, model.rt.device)
    resid, delta = model.forward(batch, cache)
    logits = model.logits(resid, delta, batch.want_rows) if batch.num_want else None
    for entry in entries:
        cache.commit(entry.request, len(entry.tokens))
    if check_errors:
        model.rt.ops.check_device_errors(model.rt.device)
    return logits
