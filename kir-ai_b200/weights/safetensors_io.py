"""Reader and writer of the safetensors container, written from the format.

A file is an 8-byte little-endian header length, a JSON header that maps each
tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets
relative to the first byte after the header), and the payload.  The checks
mirror the reference's loader (crates/llm-backend/src/core/safetensors.rs:151-303
header, :1395-1434 per-tensor offsets; 64 MiB header cap at
crates/llm-backend/src/core/safetensors/header.rs:3-44).  A folder holds either
``model.safetensors`` or ``model.safetensors.index.json`` with a ``weight_map``
from tensor name to shard file (crates/llm-models/src/safetensors.rs:11-116),
whose shard names may not leave the folder.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, Mapping, Tuple

import torch

MAX_HEADER_BYTES = 64 * 1024 * 1024

_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F64": (torch.float64, 8),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {dtype: name for name, (dtype, _) in _DTYPES.items()}


class SafetensorsError(ValueError):
    """A malformed or unreadable safetensors file; ``code`` as in the reference
    (``model_integrity_failed``, ``model_artifact_missing``, ``unsupported_capability``)."""

    def __init__(self, code: str, message: str):
        super().__init__(f"{code}: {message}")
        self.code = code


@dataclass(frozen=True)
class TensorEntry:
    dtype: str
    shape: Tuple[int, ...]
    begin: int
    end: int


def parse_header(blob: bytes, payload_bytes: int, where: str) -> Dict[str, TensorEntry]:
    """Turns the JSON header into entries, checking every offset against the payload."""
    try:
        raw = json.loads(blob.decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError) as err:
        raise SafetensorsError("model_integrity_failed", f"{where}: header is not valid JSON ({err})") from None
    if not isinstance(raw, dict):
        raise SafetensorsError("model_integrity_failed", f"{where}: header must be a JSON object")
    entries: Dict[str, TensorEntry] = {}
    for name, item in raw.items():
        if name == "__metadata__":
            continue
        if not isinstance(item, dict):
            raise SafetensorsError("model_integrity_failed", f"{where}: entry `{name}` is not an object")
        for key in ("dtype", "shape", "data_offsets"):
            if key not in item:
                raise SafetensorsError("model_integrity_failed", f"{where}: tensor `{name}` missing {key}")
        dtype, shape, offsets = item["dtype"], item["shape"], item["data_offsets"]
        if dtype not in _DTYPES:
            raise SafetensorsError("unsupported_capability", f"{where}: tensor `{name}` has unsupported dtype {dtype}")
        if not (isinstance(shape, list) and all(isinstance(n, int) and not isinstance(n, bool) and n >= 0 for n in shape)):
            raise SafetensorsError("model_integrity_failed", f"{where}: tensor `{name}` has a bad shape {shape!r}")
        if not (isinstance(offsets, list) and len(offsets) == 2 and all(isinstance(n, int) for n in offsets)):
            raise SafetensorsError("model_integrity_failed", f"{where}: tensor `{name}` has bad data_offsets")
        begin, end = offsets
        if begin < 0 or end < begin:
            raise SafetensorsError("model_integrity_failed", f"{where}: tensor `{name}` has inverted data_offsets")
        if end > payload_bytes:
            raise SafetensorsError("model_integrity_failed", f"{where}: tensor `{name}` data_offsets run past the payload")
        count = 1
        for n in shape:
            count *= n
        if count * _DTYPES[dtype][1] != end - begin:
            raise SafetensorsError(
                "model_integrity_failed",
                f"{where}: tensor `{name}` shape {shape} of {dtype} does not fill its {end - begin} bytes",
            )
        entries[name] = TensorEntry(dtype, tuple(shape), begin, end)
    if not entries:
        raise SafetensorsError("model_integrity_failed", f"{where}: file holds no tensors")
    return entries


class SafetensorsFile:
    """One memory-mapped safetensors file; tensors are read lazily by name."""

    def __init__(self, path: str | os.PathLike):
        self.path = os.fspath(path)
        try:
            self._handle = open(self.path, "rb")
        except FileNotFoundError:
            raise SafetensorsError("model_artifact_missing", f"{self.path}: no such file") from None
        size = os.fstat(self._handle.fileno()).st_size
        if size < 8:
            raise SafetensorsError("model_integrity_failed", f"{self.path}: missing the 8-byte header length")
        (header_len,) = struct.unpack("<Q", self._handle.read(8))
        if header_len > MAX_HEADER_BYTES:
            raise SafetensorsError("model_integrity_failed", f"{self.path}: header of {header_len} bytes exceeds 64 MiB")
        if 8 + header_len > size:
            raise SafetensorsError("model_integrity_failed", f"{self.path}: header runs past the end of the file")
        blob = self._handle.read(header_len)
        self._data_start = 8 + header_len
        self.entries = parse_header(blob, size - self._data_start, self.path)
        self._map = mmap.mmap(self._handle.fileno(), 0, access=mmap.ACCESS_READ)

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor over the mapped bytes of ``name`` (read-only memory: copy or move it)."""
        entry = self.entries[name]
        dtype, _ = _DTYPES[entry.dtype]
        if entry.end == entry.begin:
            return torch.empty(entry.shape, dtype=dtype)
        view = memoryview(self._map)[self._data_start + entry.begin : self._data_start + entry.end]
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the buffer is not writable
            flat = torch.frombuffer(view, dtype=dtype)
        return flat.reshape(entry.shape)

    def close(self) -> None:
        # Tensors handed out keep views of the map alive; only drop our own references.
        self._map = None
        self._handle.close()


class ModelFiles:
    """The tensors of a model folder, by name, across one file or indexed shards."""

    def __init__(self, model_dir: str | os.PathLike):
        self.model_dir = os.fspath(model_dir)
        index_path = os.path.join(self.model_dir, "model.safetensors.index.json")
        single_path = os.path.join(self.model_dir, "model.safetensors")
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        if os.path.exists(index_path):
            try:
                with open(index_path, "r", encoding="utf-8") as handle:
                    index = json.load(handle)
                weight_map = index["weight_map"]
                assert isinstance(weight_map, dict)
            except (json.JSONDecodeError, KeyError, AssertionError) as err:
                raise SafetensorsError("model_integrity_failed", f"{index_path}: bad index ({err})") from None
            root = os.path.realpath(self.model_dir)
            for name, shard in weight_map.items():
                if not isinstance(shard, str) or os.path.isabs(shard) or ".." in shard.replace("\\", "/").split("/"):
                    raise SafetensorsError("model_integrity_failed", f"{index_path}: unsafe shard path {shard!r}")
                full = os.path.realpath(os.path.join(self.model_dir, shard))
                if os.path.commonpath([root, full]) != root:
                    raise SafetensorsError("model_integrity_failed", f"{index_path}: shard {shard!r} escapes the model folder")
                if shard not in self._files:
                    self._files[shard] = SafetensorsFile(full)
                if name not in self._files[shard].entries:
                    raise SafetensorsError("model_integrity_failed", f"{index_path}: `{name}` is not in shard {shard}")
                self._where[name] = shard
        elif os.path.exists(single_path):
            self._files["model.safetensors"] = SafetensorsFile(single_path)
            for name in self._files["model.safetensors"].names():
                self._where[name] = "model.safetensors"
        else:
            raise SafetensorsError(
                "model_artifact_missing",
                f"{self.model_dir}: neither model.safetensors nor model.safetensors.index.json",
            )

    def names(self) -> Iterable[str]:
        return self._where.keys()

    def entry(self, name: str) -> TensorEntry:
        return self._files[self._where[name]].entries[name]

    def tensor(self, name: str) -> torch.Tensor:
        return self._files[self._where[name]].tensor(name)


def write_safetensors(path: str | os.PathLike, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] | None = None) -> None:
    """Writes ``tensors`` (CPU, any of the supported dtypes) as one safetensors file."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors.keys())
    for name in order:
        tensor = tensors[name]
        if tensor.dtype not in _NAMES:
            raise SafetensorsError("unsupported_capability", f"tensor `{name}` has unsupported dtype {tensor.dtype}")
        nbytes = tensor.numel() * tensor.element_size()
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(blob)))
        handle.write(blob)
        for name in order:
            tensor = tensors[name].detach().cpu().contiguous()
            handle.write(tensor.view(torch.uint8).numpy().tobytes() if tensor.numel() else b"")
