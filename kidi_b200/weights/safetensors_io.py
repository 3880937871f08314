"""A bounds-checked reader and a writer for the safetensors format.

Format and checks follow the reference's reader
(src/kidi/checkpoint/safetensors/mapped.h:36-51,135-139,574-639): a little-endian
u64 header length, a JSON header {name: {dtype, shape, data_offsets}} in which
`__metadata__` is skipped, then the payload; limits of 8 dimensions, one million
tensors and (here) a 100 MiB header; every entry must satisfy
`end - begin == numel * itemsize`, lie inside the payload and have no negative
dimension; duplicate names are rejected by the JSON parser hook, and so are two entries
whose byte ranges overlap. The file is mapped
read-only and tensors are views into the mapping
(src/kidi/checkpoint/safetensors/mapped.h:388-417). The writer pads the header to 8
bytes like src/kidi/checkpoint/weights.cpp:148-198.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Mapping, Tuple

import numpy as np
import torch

from ..errors import invalid_manifest, io_error

MAX_HEADER_BYTES = 100 << 20
MAX_TENSORS = 1_000_000
MAX_DIMENSIONS = 8

# safetensors dtype string -> (torch dtype, numpy carrier dtype, itemsize)
_DTYPES = {
    "F32": (torch.float32, np.dtype("<f4"), 4),
    "BF16": (torch.bfloat16, np.dtype("<u2"), 2),
    "F16": (torch.float16, np.dtype("<f2"), 2),
    "F64": (torch.float64, np.dtype("<f8"), 8),
    "I32": (torch.int32, np.dtype("<i4"), 4),
    "I64": (torch.int64, np.dtype("<i8"), 8),
    "U8": (torch.uint8, np.dtype("u1"), 1),
    "I8": (torch.int8, np.dtype("i1"), 1),
}
_NAMES = {torch_dtype: name for name, (torch_dtype, _, _) in _DTYPES.items()}


class TensorEntry:
    __slots__ = ("name", "dtype", "shape", "begin", "end")

    def __init__(self, name: str, dtype: str, shape: Tuple[int, ...], begin: int, end: int):
        self.name, self.dtype, self.shape, self.begin, self.end = name, dtype, shape, begin, end


def _reject_duplicates(pairs):
    seen = {}
    for key, value in pairs:
        if key in seen:
            raise invalid_manifest(f"safetensors header names '{key}' twice")
        seen[key] = value
    return seen


class SafetensorsFile:
    """A mapped safetensors file; `tensor(name)` returns a read-only view."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._handle = open(path, "rb")
            size = os.fstat(self._handle.fileno()).st_size
        except OSError as error:
            raise io_error(f"cannot open {path}: {error}") from None
        if size < 8:
            raise invalid_manifest(f"{path}: file too small for a safetensors header")
        self._map = mmap.mmap(self._handle.fileno(), 0, access=mmap.ACCESS_READ)
        (header_length,) = struct.unpack("<Q", self._map[:8])
        if header_length > MAX_HEADER_BYTES or 8 + header_length > size:
            raise invalid_manifest(f"{path}: header length {header_length} exceeds the file or the limit")
        try:
            header = json.loads(self._map[8:8 + header_length].decode("utf-8"),
                                object_pairs_hook=_reject_duplicates)
        except (UnicodeDecodeError, json.JSONDecodeError) as error:
            raise invalid_manifest(f"{path}: malformed safetensors header: {error}") from None
        if not isinstance(header, dict):
            raise invalid_manifest(f"{path}: safetensors header must be an object")
        self._payload_offset = 8 + header_length
        payload = size - self._payload_offset
        self.entries: Dict[str, TensorEntry] = {}
        if len(header) > MAX_TENSORS:
            raise invalid_manifest(f"{path}: more than {MAX_TENSORS} tensors")
        for name, item in header.items():
            if name == "__metadata__":
                continue
            if not isinstance(item, dict) or not {"dtype", "shape", "data_offsets"} <= set(item):
                raise invalid_manifest(f"{path}: entry '{name}' lacks dtype, shape or data_offsets")
            dtype, shape, offsets = item["dtype"], item["shape"], item["data_offsets"]
            if dtype not in _DTYPES:
                raise invalid_manifest(f"{path}: tensor '{name}' has unknown dtype '{dtype}'")
            if (not isinstance(shape, list) or len(shape) > MAX_DIMENSIONS
                    or not all(isinstance(d, int) and not isinstance(d, bool) and d >= 0 for d in shape)):
                raise invalid_manifest(f"{path}: tensor '{name}' has an invalid shape {shape!r}")
            if (not isinstance(offsets, list) or len(offsets) != 2
                    or not all(isinstance(o, int) and not isinstance(o, bool) for o in offsets)):
                raise invalid_manifest(f"{path}: tensor '{name}' has invalid data_offsets")
            begin, end = offsets
            numel = 1
            for dimension in shape:
                numel *= dimension
            if begin < 0 or end < begin or end > payload or end - begin != numel * _DTYPES[dtype][2]:
                raise invalid_manifest(
                    f"{path}: tensor '{name}' spans bytes [{begin}, {end}) but needs "
                    f"{numel * _DTYPES[dtype][2]} inside a payload of {payload}")
            self.entries[name] = TensorEntry(name, dtype, tuple(shape), begin, end)
        # No two tensors may share payload bytes: sorted by their first byte, each must end
        # before the next begins (empty tensors take no bytes and cannot overlap anything).
        spans = sorted((entry.begin, entry.end, entry.name) for entry in self.entries.values()
                       if entry.end > entry.begin)
        for (_, end, name), (begin, _, other) in zip(spans, spans[1:]):
            if begin < end:
                raise invalid_manifest(f"{path}: tensors '{name}' and '{other}' overlap in the payload")

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name].shape

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name].dtype][0]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor viewing the mapping (do not write to it)."""
        entry = self.entries[name]
        torch_dtype, carrier, itemsize = _DTYPES[entry.dtype]
        count = (entry.end - entry.begin) // itemsize
        if count == 0:
            return torch.empty(entry.shape, dtype=torch_dtype)
        array = np.frombuffer(self._map, dtype=carrier, count=count, offset=self._payload_offset + entry.begin)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the view is read-only by contract
            flat = torch.from_numpy(array)
        if torch_dtype == torch.bfloat16:
            flat = flat.view(torch.bfloat16)
        return flat.reshape(entry.shape)

    def close(self) -> None:
        # Views keep the mapping alive through numpy's buffer reference; closing the
        # handle alone is always safe.
        try:
            self._handle.close()
        except OSError:
            pass


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] = None) -> None:
    """Writes tensors (CPU, contiguous) in the order given; refuses to overwrite."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    ordered = []
    for name, tensor in tensors.items():
        if tensor.dtype not in _NAMES:
            raise invalid_manifest(f"tensor '{name}' has a dtype safetensors cannot hold: {tensor.dtype}")
        tensor = tensor.detach().cpu().contiguous()
        nbytes = tensor.numel() * tensor.element_size()
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        ordered.append(tensor)
    encoded = json.dumps(header, separators=(",", ":")).encode("utf-8")
    encoded += b" " * (-len(encoded) % 8)
    try:
        with open(path, "xb") as handle:
            handle.write(struct.pack("<Q", len(encoded)))
            handle.write(encoded)
            for tensor in ordered:
                if tensor.numel() == 0:
                    continue
                carrier = tensor.view(torch.uint16) if tensor.dtype == torch.bfloat16 else tensor
                handle.write(carrier.numpy().tobytes() if carrier.numel() < (1 << 24) else memoryview(carrier.numpy()).cast("B"))
    except FileExistsError:
        raise io_error(f"{path} exists already") from None
    except OSError as error:
        raise io_error(f"cannot write {path}: {error}") from None
