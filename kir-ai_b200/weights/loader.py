"""Loads the tensors a model asks for, by name, and checks them all at once.

``check_and_open`` compares the names and shapes that the model's parts declare
(``weight_specs``) with what the model folder holds and raises one
``WeightError`` that lists every missing tensor, every unexpected tensor and
every wrong shape or dtype family.  The reference checks presence before
loading (crates/llm-models/src/qwen.rs:215-260) and shapes at use
(crates/llm-backend/src/core/qwen/ops/moe.rs:74-82); here both happen up front.

Dtype policy: a floating tensor stored in bfloat16 stays bfloat16 and one
stored in 32-bit stays 32-bit on the way in; integer tables become int32.  What
a part does with a tensor is the part's business (a bf16 linear layer needs a
bf16 matrix, norm weights are always widened to 32-bit, the true 32-bit path
widens everything).
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..parts.base import WeightSpec
from .safetensors_io import ModelFiles

_FLOAT = {"F32", "BF16", "F16", "F64"}
_INT = {"I64", "I32", "I16", "I8", "U8"}


class WeightError(ValueError):
    """The model folder does not hold what the model needs."""

    def __init__(self, missing, unexpected, wrong):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong = list(wrong)
        lines = ["model weights do not match the configuration:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong:
            lines.append(f"  wrong shape or type ({len(self.wrong)}):")
            lines.extend(f"    {item}" for item in self.wrong)
        super().__init__("\n".join(lines))


class WeightSource:
    """Hands tensors to the parts and remembers device copies, so that two parts
    that name the same tensor (tied embedding and output head) share one buffer."""

    def __init__(self, tensors, device: torch.device):
        self._tensors = tensors  # ModelFiles or a mapping of name -> tensor
        self.device = torch.device(device)
        self._device_copies: Dict[tuple, torch.Tensor] = {}

    def stored(self, name: str) -> torch.Tensor:
        """The tensor as stored (CPU for a model folder), integers as int32."""
        tensor = self._tensors.tensor(name) if hasattr(self._tensors, "tensor") else self._tensors[name]
        if not tensor.is_floating_point():
            tensor = tensor.to(torch.int32)
        elif tensor.dtype not in (torch.float32, torch.bfloat16):
            tensor = tensor.to(torch.float32)
        return tensor

    def on_device(self, name: str, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """A contiguous device copy in ``dtype`` (default: as stored), shared between callers."""
        stored = self.stored(name)
        dtype = dtype or stored.dtype
        key = (name, dtype)
        if key not in self._device_copies:
            self._device_copies[key] = stored.to(device=self.device, dtype=dtype).contiguous()
        return self._device_copies[key]

    def shared(self, key: tuple, make):
        """What ``make()`` returns, made once per ``key`` and handed to every caller: parts that read the same
        stored tensor in the same derived form (a tied table in a kernel's own layout) hold one copy."""
        if key not in self._device_copies:
            self._device_copies[key] = make()
        return self._device_copies[key]

    def forget(self) -> None:
        """Drops the bookkeeping (not the tensors that parts hold)."""
        self._device_copies.clear()


def check(specs: Mapping[str, WeightSpec], present: Mapping[str, tuple], ignorable=()) -> None:
    """``present`` maps name -> (dtype name, shape).  Raises WeightError on any mismatch.  Names in ``ignorable``
    may be present without being wanted: a tied checkpoint that still ships its output head loads in the
    reference, which only asks for the names it needs (crates/llm-models/src/qwen.rs:215-260)."""
    missing = [name for name in specs if name not in present]
    unexpected = [name for name in present if name not in specs and name not in set(ignorable)]
    wrong = []
    for name, spec in specs.items():
        if name not in present:
            continue
        dtype, shape = present[name]
        if tuple(shape) != tuple(spec.shape):
            wrong.append(f"{name}: shape {list(shape)}, expected {list(spec.shape)}")
        elif spec.role == "int_table" and dtype not in _INT:
            wrong.append(f"{name}: dtype {dtype}, expected an integer table")
        elif spec.role != "int_table" and dtype not in _FLOAT:
            wrong.append(f"{name}: dtype {dtype}, expected a floating tensor")
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong)


_TORCH_NAMES = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16", torch.float64: "F64",
                torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8"}


def open_checked(model_dir: str, specs: Mapping[str, WeightSpec], device, ignorable=()) -> WeightSource:
    """Opens a model folder, checks it against ``specs`` and returns the source for ``load``."""
    files = ModelFiles(model_dir)
    present = {name: (files.entry(name).dtype, files.entry(name).shape) for name in files.names()}
    check(specs, present, ignorable)
    return WeightSource(files, device)


def from_tensors(tensors: Mapping[str, torch.Tensor], specs: Mapping[str, WeightSpec], device, ignorable=()) -> WeightSource:
    """The same check for tensors already in memory (random weights made on the device)."""
    present = {name: (_TORCH_NAMES.get(t.dtype, str(t.dtype)), tuple(t.shape)) for name, t in tensors.items()}
    check(specs, present, ignorable)
    return WeightSource(dict(tensors), device)
