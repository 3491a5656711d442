"""Turns logits into tokens on the device: greedy rows by argmax (lowest index on
ties), the others by nucleus sampling with the row's draw."""
from __future__ import annotations

from typing import Sequence

import torch


def sample(ops, logits: torch.Tensor, temperatures: Sequence[float], top_ps: Sequence[float],
           draws: Sequence[float]) -> torch.Tensor:
    """One token id per row of ``logits`` [rows, vocab] (int32, on the device)."""
    if all(t == 0.0 for t in temperatures):
        return ops.argmax_rows(logits)
    host = torch.tensor([list(temperatures), list(top_ps), list(draws)], dtype=torch.float32)
    if logits.is_cuda:
        host = host.pin_memory()
    dev = host.to(logits.device, non_blocking=True)
    return ops.sample_rows(logits, dev[0], dev[1], dev[2])
