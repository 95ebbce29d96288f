"""Reading and writing the safetensors container: a directory of named tensors.

File layout: 8 bytes little-endian header length N, N bytes of JSON
`{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}`,
then the raw little-endian tensor bytes, offsets relative to the end of the header.

This plays the role of the reference's GGUF reader (src/gguf.zig:286-478): the header is
parsed once, tensor data stay on disk (memory-mapped here, `pread` on demand there) and
are found by name through a hash map, not a scan (src/gguf.zig:232-237).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, Tuple

import torch

_DTYPES = {
    "F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int
    end: int
    file: str


class SafetensorsFile:
    """One memory-mapped .safetensors file."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
        except OSError:
            raise SafetensorsError(f"{path}: no such file") from None
        if size < 8:
            raise SafetensorsError(f"{path}: truncated (no header length)")
        self._fh = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file size {size}")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        self.data_start = 8 + hlen
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            try:
                dtype, shape = info["dtype"], tuple(int(s) for s in info["shape"])
                begin, end = (int(o) for o in info["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for tensor {name!r}") from None
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dtype}")
            n = 1
            for s in shape:
                n *= s
            want = n * torch.empty((), dtype=_DTYPES[dtype]).element_size()
            if end - begin != want or begin < 0 or self.data_start + end > size:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} of shape {list(shape)} {dtype} needs {want} bytes but its "
                    f"offsets [{begin}, {end}) give {end - begin} (file holds {size - self.data_start} data bytes)")
            self.entries[name] = TensorEntry(name, dtype, shape, begin, end, path)
        # A private copy-on-write map: tensors made from it are writable views that never
        # touch the file.
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_COPY) if size > 0 else None

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        dtype = _DTYPES[e.dtype]
        n = 1
        for s in e.shape:
            n *= s
        if n == 0:
            return torch.empty(e.shape, dtype=dtype)
        t = torch.frombuffer(self._map, dtype=dtype, count=n, offset=self.data_start + e.begin)
        return t.view(e.shape)


class TensorDirectory:
    """All named tensors of a model folder (one file, or shards listed by an index)."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        files = []
        if os.path.isfile(single):
            files = [single]
        elif os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as f:
                weight_map = json.load(f).get("weight_map", {})
            files = sorted({os.path.join(model_dir, v) for v in weight_map.values()})
        if not files:
            raise SafetensorsError(f"{model_dir}: no model.safetensors (or model.safetensors.index.json) found")
        self.files = [SafetensorsFile(p) for p in files]
        self.where: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for name in f.entries:
                self.where[name] = f

    def names(self) -> Iterable[str]:
        return self.where.keys()

    def entry(self, name: str) -> TensorEntry:
        return self.where[name].entries[name]

    def tensor(self, name: str) -> torch.Tensor:
        return self.where[name].tensor(name)

    def __contains__(self, name: str) -> bool:
        return name in self.where


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] | None = None) -> None:
    """Write `tensors` (CPU, contiguous) to `path`, names in sorted order."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot write tensor {name!r} of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous().reshape(-1)
            if t.numel():
                f.write(memoryview(t.view(torch.uint8).numpy()))
