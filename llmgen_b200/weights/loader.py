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

import fnmatch
from typing import Dict, Iterable, List, Sequence, Tuple

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


class PinnedStage:
    """Host-to-device copies of tensors that live in a memory-mapped file: through two pinned buffers of
    32 MiB used in turn, so that the copy engine reads page-locked memory while the host fills the other
    buffer from the file (the reference stages its uploads the same way, src/memory/manager.zig:263-300).
    A pageable `.to(device)` would have the driver stage every tensor through a small buffer of its own,
    one synchronous piece at a time."""

    CHUNK = 32 << 20

    def __init__(self, device):
        self.device = torch.device(device)
        self._buffers = None
        self._events = [None, None]
        self._turn = 0
        self.bytes_moved = 0

    def upload(self, src: torch.Tensor) -> torch.Tensor:
        """A device tensor with the values (and dtype) of the host tensor `src`."""
        if self.device.type != "cuda" or src.is_cuda or src.numel() * src.element_size() < (1 << 20):
            return src.to(self.device)
        if self._buffers is None:
            self._buffers = [torch.empty(self.CHUNK, dtype=torch.uint8).pin_memory() for _ in range(2)]
        src = src.contiguous()
        out = torch.empty(src.shape, dtype=src.dtype, device=self.device)
        from_bytes = src.reshape(-1).view(torch.uint8)
        to_bytes = out.reshape(-1).view(torch.uint8)
        total = from_bytes.numel()
        for at in range(0, total, self.CHUNK):
            turn = self._turn
            self._turn ^= 1
            if self._events[turn] is not None:
                self._events[turn].synchronize()         # the copy that last read this buffer has finished
            n = min(self.CHUNK, total - at)
            self._buffers[turn][:n].copy_(from_bytes[at:at + n])
            to_bytes[at:at + n].copy_(self._buffers[turn][:n], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self._events[turn] = ev
        self.bytes_moved += total
        return out

    def close(self) -> None:
        for ev in self._events:
            if ev is not None:
                ev.synchronize()
        self._buffers, self._events = None, [None, None]


class WeightStore:
    """Checked access to a folder's tensors; uploads each name once."""

    def __init__(self, directory, decls: Dict[str, WeightDecl]):
        self.directory = directory
        self.decls = decls
        self._device_cache: Dict[tuple, torch.Tensor] = {}
        self._stages: Dict[str, PinnedStage] = {}

    def _stage(self, device) -> PinnedStage:
        key = str(device)
        if key not in self._stages:
            self._stages[key] = PinnedStage(device)
        return self._stages[key]

    def host_tensor(self, name: str) -> torch.Tensor:
        if name not in self.decls:
            raise WeightError(f"tensor {name!r} was not declared by any part")
        return self.directory.tensor(name)

    def device_tensor(self, name: str, compute_dtype: torch.dtype, device, keep: bool = True) -> torch.Tensor:
        """The tensor on the device in the dtype its kind asks for.  `keep=False`: the caller packs it into a
        tensor of its own and nobody else reads it, so the store does not hold on to the upload."""
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
        if key in self._device_cache:
            return self._device_cache[key]
        # the file's bytes go up as they are; a change of dtype (an exact widening) happens on the device
        t = self._stage(device).upload(self.directory.tensor(name)).to(dtype).contiguous()
        if keep:
            self._device_cache[key] = t
        return t

    def release(self) -> None:
        """Drop the upload cache and the pinned buffers (the parts keep what they took)."""
        self._device_cache.clear()
        for stage in self._stages.values():
            stage.close()
        self._stages.clear()


def validate(directory, decls: Dict[str, WeightDecl], where: str, ignorable: Sequence[str] = (),
             same_as: Sequence[Tuple[str, str]] = ()) -> None:
    """One `WeightError` for everything that does not fit.  `ignorable`: shell patterns of tensors the folder
    may carry unread; `same_as`: (such a tensor, a declared one) whose values must then be equal, as for the
    output matrix that exports of tied models carry beside the table it copies."""
    present = set(directory.names())
    missing = [n for n in decls if n not in present]
    unexpected = sorted(n for n in present - set(decls) if not any(fnmatch.fnmatchcase(n, pat) for pat in ignorable))
    wrong: List[str] = []
    for extra, declared in same_as:
        if extra in present and extra not in decls and declared in present:
            a, b = directory.entry(extra), directory.entry(declared)
            if tuple(a.shape) != tuple(b.shape) or a.dtype != b.dtype or not torch.equal(directory.tensor(extra), directory.tensor(declared)):
                wrong.append(f"{extra}: the model reads {declared} in its place (tied), but the two differ")
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


def open_weights(model_dir: str, decls: Iterable[WeightDecl], ignorable: Sequence[str] = (),
                 same_as: Sequence[Tuple[str, str]] = ()) -> WeightStore:
    merged = check_declarations(list(decls))
    try:
        directory = TensorDirectory(model_dir)
    except SafetensorsError as e:
        raise WeightError(str(e)) from None
    validate(directory, merged, model_dir, ignorable, same_as)
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
