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


_CODES = {1: "model_artifact_missing", 2: "model_integrity_failed", 3: "unsupported_capability"}
_native_library = None


def _native():
    """The host library with the native reader (csrc/safetensors_reader.cpp), its functions typed."""
    global _native_library
    if _native_library is None:
        import ctypes

        from ..csrc import build as _build

        lib = ctypes.CDLL(_build.build_host())
        lib.kirai_st_open.restype = ctypes.c_void_p
        lib.kirai_st_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_int), ctypes.c_char_p, ctypes.c_int]
        lib.kirai_st_close.argtypes = [ctypes.c_void_p]
        lib.kirai_st_count.argtypes = [ctypes.c_void_p]
        lib.kirai_st_entry.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_int,
                                       ctypes.POINTER(ctypes.c_long), ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_long),
                                       ctypes.POINTER(ctypes.c_long)]
        lib.kirai_st_payload.restype = ctypes.c_void_p
        lib.kirai_st_payload.argtypes = [ctypes.c_void_p]
        _native_library = lib
    return _native_library


class SafetensorsFile:
    """One memory-mapped safetensors file; tensors are read lazily by name.

    The file is mapped and its header parsed and checked in native code (csrc/safetensors_reader.cpp); with
    ``native=False`` the Python reader of this module does the same (the tests hold the two against each other)."""

    def __init__(self, path: str | os.PathLike, native: bool = True):
        self.path = os.fspath(path)
        self._native_handle = None
        if native:
            self._open_native()
            return
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

    def _open_native(self) -> None:
        import ctypes

        lib = _native()
        code = ctypes.c_int(0)
        message = ctypes.create_string_buffer(1024)
        handle = lib.kirai_st_open(self.path.encode("utf-8"), ctypes.byref(code), message, len(message))
        if not handle:
            text = message.value.decode("utf-8", "replace")
            raise SafetensorsError(_CODES.get(code.value, "model_integrity_failed"), text)
        self._native_handle = handle
        self._payload = lib.kirai_st_payload(handle)
        self.entries = {}
        name, dtype = ctypes.create_string_buffer(4096), ctypes.create_string_buffer(16)
        shape, rank = (ctypes.c_long * 16)(), ctypes.c_int(0)
        begin, end = ctypes.c_long(0), ctypes.c_long(0)
        for index in range(lib.kirai_st_count(handle)):
            status = lib.kirai_st_entry(handle, index, name, len(name), dtype, len(dtype), shape, ctypes.byref(rank),
                                        ctypes.byref(begin), ctypes.byref(end))
            if status != 0:
                raise SafetensorsError("model_integrity_failed", f"{self.path}: a tensor name or shape is too long to read")
            try:
                key = name.value.decode("utf-8")
            except UnicodeDecodeError:
                raise SafetensorsError("model_integrity_failed", f"{self.path}: a tensor name is not valid UTF-8") from None
            self.entries[key] = TensorEntry(dtype.value.decode("ascii"), tuple(shape[: rank.value]), begin.value, end.value)

    def __del__(self):
        handle, self._native_handle = getattr(self, "_native_handle", None), None
        if handle and _native_library is not None:
            _native_library.kirai_st_close(handle)

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor over the mapped bytes of ``name`` (read-only memory: copy or move it)."""
        entry = self.entries[name]
        dtype, _ = _DTYPES[entry.dtype]
        if entry.end == entry.begin:
            return torch.empty(entry.shape, dtype=dtype)
        import warnings

        if self._native_handle is not None:
            import ctypes

            view = (ctypes.c_ubyte * (entry.end - entry.begin)).from_address(self._payload + entry.begin)
            view._owner = self  # the tensor keeps the view, and the view keeps the mapping, alive
        else:
            view = memoryview(self._map)[self._data_start + entry.begin : self._data_start + entry.end]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the buffer is not writable
            flat = torch.frombuffer(view, dtype=dtype)
        return flat.reshape(entry.shape)

    def close(self) -> None:
        # Tensors handed out keep views of the map alive; only drop our own references.  (The native mapping
        # goes when the last tensor over it and this object are gone.)
        if self._native_handle is None:
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
            handle.write(tensor.reshape(-1).view(torch.uint8).numpy().tobytes() if tensor.numel() else b"")
