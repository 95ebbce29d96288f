"""Weights by tensor name: check the model folder against what the model declares, then
hand tensors to the parts.

Every part declares the tensors it reads (`WeightDecl`: name, shape, role).  `open_weights`
compares those declarations with the folder's tensor directory and raises ONE
`WeightError` that lists every missing tensor, every unexpected tensor and every wrong
shape or unsupported dtype.  The reference fails on the first missing name
(`error.MissingWeight`, src/module/trace.zig:47-59) and checks dtypes at upload
(`error.UnsupportedWeightDtype`, src/memory/manager.zig:215-218).

Dtypes on the device (`device_tensor`): matrices and embedding tables take the engine's
compute dtype (bfloat16, or float32 for the true 32-bit path, an exact widening of
bfloat16 storage); vectors such as norm gains are float32 whatever the file holds (again an
exact widening); integer tables become int32.  Tensors of the same name are uploaded once
and shared (tied embeddings; src/memory/manager.zig:269-279).
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Sequence

import torch

from ..parts.spec import INT_TABLE, MATRIX, VECTOR, WeightDecl
from .safetensors_io import SafetensorsError, TensorDirectory

_FLOAT_DTYPES = ("F32", "BF16", "F16")
_INT_DTYPES = ("I64", "I32", "I16", "I8", "U8")


class WeightError(ValueError):
    """The model folder does not hold the tensors the model declares."""


def check_declarations(decls: Sequence[WeightDecl]) -> Dict[str, WeightDecl]:
    """Merge declarations by name; the same name twice must agree in shape (tying)."""
    merged: Dict[str, WeightDecl] = {}
    for d in decls:
        if d.name in merged:
            if tuple(merged[d.name].shape) != tuple(d.shape):
                raise WeightError(f"tensor {d.name!r} is declared with shapes "
                                  f"{list(merged[d.name].shape)} and {list(d.shape)}")
        else:
            merged[d.name] = d
    return merged


class WeightStore:
    """Checked access to a folder's tensors; uploads each name once."""

    def __init__(self, directory, decls: Dict[str, WeightDecl]):
        self.directory = directory
        self.decls = decls
        self._device_cache: Dict[tuple, torch.Tensor] = {}

    def host_tensor(self, name: str) -> torch.Tensor:
        if name not in self.decls:
            raise WeightError(f"tensor {name!r} was not declared by any part")
        return self.directory.tensor(name)

    def device_tensor(self, name: str, compute_dtype: torch.dtype, device) -> torch.Tensor:
        decl = self.decls.get(name)
        if decl is None:
            raise WeightError(f"tensor {name!r} was not declared by any part")
        if decl.kind == MATRIX:
            dtype = compute_dtype
        elif decl.kind == VECTOR:
            dtype = torch.float32
        else:
            dtype = torch.int32
        key = (name, dtype, str(device))
        if key not in self._device_cache:
            self._device_cache[key] = self.directory.tensor(name).to(device=device, dtype=dtype).contiguous()
        return self._device_cache[key]

    def release(self) -> None:
        """Drop the upload cache (the parts keep what they took)."""
        self._device_cache.clear()


def validate(directory, decls: Dict[str, WeightDecl], where: str) -> None:
    present = set(directory.names())
    missing = [n for n in decls if n not in present]
    unexpected = sorted(present - set(decls))
    wrong: List[str] = []
    for name, d in decls.items():
        if name not in present:
            continue
        e = directory.entry(name)
        if tuple(e.shape) != tuple(d.shape):
            wrong.append(f"{name}: file has {list(e.shape)}, model needs {list(d.shape)}")
        allowed = _INT_DTYPES if d.kind == INT_TABLE else _FLOAT_DTYPES
        if e.dtype not in allowed:
            wrong.append(f"{name}: dtype {e.dtype} is not supported here (allowed: {', '.join(allowed)})")
    if missing or unexpected or wrong:
        parts = [f"{where}: the tensors do not match the model"]
        if missing:
            parts.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            parts.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            parts.append(f"  wrong shape or dtype ({len(wrong)}): " + "; ".join(wrong))
        raise WeightError("\n".join(parts))


def open_weights(model_dir: str, decls: Iterable[WeightDecl]) -> WeightStore:
    merged = check_declarations(list(decls))
    try:
        directory = TensorDirectory(model_dir)
    except SafetensorsError as e:
        raise WeightError(str(e)) from None
    validate(directory, merged, model_dir)
    return WeightStore(directory, merged)


class DictDirectory:
    """A tensor directory over an in-memory dict (random weights without a folder)."""

    class _Entry:
        def __init__(self, t: torch.Tensor):
            self.shape = tuple(t.shape)
            self.dtype = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16",
                          torch.int32: "I32", torch.int64: "I64"}.get(t.dtype, str(t.dtype))

    def __init__(self, tensors: Dict[str, torch.Tensor]):
        self.tensors = tensors

    def names(self):
        return self.tensors.keys()

    def entry(self, name):
        return DictDirectory._Entry(self.tensors[name])

    def tensor(self, name):
        return self.tensors[name]


def weights_from_dict(tensors: Dict[str, torch.Tensor], decls: Iterable[WeightDecl]) -> WeightStore:
    merged = check_declarations(list(decls))
    directory = DictDirectory(tensors)
    validate(directory, merged, "<in-memory tensors>")
    return WeightStore(directory, merged)
