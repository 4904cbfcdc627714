"""Reading and writing the safetensors container: an 8-byte little-endian header length, a JSON
header ``{name: {dtype, shape, data_offsets}}`` and the raw little-endian tensor bytes.

Files are memory-mapped and tensors are views into the map until they are copied to the device
(the reference maps aligned files too, crates/mrun-engine/src/tensor/nuvec.rs:1081-1098).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Iterator, Tuple

import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {dtype: name for name, (dtype, _) in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """A mapped file: ``names()``, ``info(name)`` (dtype, shape) and ``tensor(name)``."""

    def __init__(self, path: str):
        self.path = path
        self._file = open(path, "rb")
        size = os.fstat(self._file.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors header")
        (length,) = struct.unpack("<Q", self._file.read(8))
        if length > size - 8:
            raise SafetensorsError(f"{path}: header length {length} exceeds the file")
        try:
            header = json.loads(self._file.read(length).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as error:
            raise SafetensorsError(f"{path}: header is not JSON: {error}") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        self._entries: Dict[str, dict] = header
        self._base = 8 + length
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        for name, entry in header.items():
            if entry.get("dtype") not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name} has unsupported dtype "
                                       f"{entry.get('dtype')}")
            begin, end = entry["data_offsets"]
            count = 1
            for extent in entry["shape"]:
                count *= extent
            if end - begin != count * _DTYPES[entry["dtype"]][1] or self._base + end > size:
                raise SafetensorsError(f"{path}: tensor {name} has inconsistent offsets")

    def names(self) -> list[str]:
        return list(self._entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        entry = self._entries[name]
        return _DTYPES[entry["dtype"]][0], tuple(entry["shape"])

    def tensor(self, name: str) -> torch.Tensor:
        entry = self._entries[name]
        dtype, _ = _DTYPES[entry["dtype"]]
        begin, end = entry["data_offsets"]
        shape = tuple(entry["shape"])
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        view = memoryview(self._map)[self._base + begin:self._base + end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the map is read-only; tensors are never written
            flat = torch.frombuffer(view, dtype=dtype)
        return flat.reshape(shape)


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]],
                      metadata: Dict[str, str] | None = None) -> None:
    """Writes ``(name, tensor)`` pairs.  The iterable is consumed twice-free: tensors are staged
    one by one, so a generator that makes them lazily keeps memory at one tensor."""
    staged: list[Tuple[str, str, Tuple[int, ...], int]] = []
    tmp = path + ".tmp"
    offset = 0
    with open(tmp + ".data", "wb") as data:
        for name, tensor in tensors:
            tensor = tensor.detach().to("cpu").contiguous()
            if tensor.dtype not in _NAMES:
                raise SafetensorsError(f"tensor {name}: dtype {tensor.dtype} cannot be stored")
            raw = tensor.reshape(-1).view(torch.uint8).numpy().tobytes() if tensor.numel() else b""
            data.write(raw)
            staged.append((name, _NAMES[tensor.dtype], tuple(tensor.shape), len(raw)))
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = metadata
    for name, dtype, shape, nbytes in staged:
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    with open(tmp, "wb") as out:
        out.write(struct.pack("<Q", len(blob)))
        out.write(blob)
        with open(tmp + ".data", "rb") as data:
            while True:
                chunk = data.read(1 << 24)
                if not chunk:
                    break
                out.write(chunk)
    os.remove(tmp + ".data")
    os.replace(tmp, path)


def open_model_files(model_dir: str) -> list[SafetensorsFile]:
    """Every ``*.safetensors`` of a folder, sorted by name; no index file is consulted
    (crates/mrun-engine/src/load.rs:179-196)."""
    names = sorted(n for n in os.listdir(model_dir) if n.endswith(".safetensors"))
    if not names:
        raise FileNotFoundError(f"no *.safetensors files in {model_dir}")
    return [SafetensorsFile(os.path.join(model_dir, n)) for n in names]


def iter_tensors(files: list[SafetensorsFile]) -> Iterator[Tuple[str, SafetensorsFile]]:
    for f in files:
        for name in f.names():
            yield name, f
