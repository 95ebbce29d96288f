"""What a step hands to the parts: packed metadata on the device, and named workspaces.

One step = one pinned host buffer filled by `StepMetaBuilder`, ONE host-to-device copy, then
kernel launches that read int32 views of the device copy (the reference's `Layout` /
`fillMeta` / `uploadMeta`, src/executor.zig:139-202, 772-861, 765-769).  Array offsets depend
only on the order and sizes of the arrays added, which depend only on (tokens, sequences) of
the step, so a CUDA graph captured for a bucket finds its inputs at the same addresses on
every replay.

Parts may add arrays of their own (`StepMetaBuilder.add`) in `prepare_step`; they read them
back by name from `StepContext.array`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch


class Workspace:
    """Named device buffers of fixed capacity; `rows` of a buffer never move.

    A buffer is created the first time its name is asked for, with room for `capacity_rows`
    rows (the engine's tokens-per-step limit by default), and later calls return views of the
    same memory: activation addresses depend on nothing but the name, which is what graph
    replay needs (the property the reference gets from its liveness plan,
    src/memory/plan.zig:121-185).
    """

    def __init__(self, device, default_rows: int):
        self.device = device
        self.default_rows = default_rows
        self._buffers: Dict[str, torch.Tensor] = {}
        self._views: Dict[Tuple, torch.Tensor] = {}   # (name, rows, cols, dtype) -> the view handed out last time
        self._retired: List[torch.Tensor] = []   # replaced buffers stay alive: captured graphs still use them
        self.frozen = False   # set while a graph is being captured: no new allocations

    def buffer(self, name: str, rows: int, cols: int, dtype: torch.dtype, capacity_rows: Optional[int] = None) -> torch.Tensor:
        # the same view object for the same request: a step asks for a few hundred, and making a
        # view costs more than finding one
        vkey = (name, rows, cols, dtype)
        view = self._views.get(vkey)
        if view is not None:
            return view
        view = self._buffer(name, rows, cols, dtype, capacity_rows)
        if len(self._views) > 4096:
            self._views.clear()
        self._views[vkey] = view
        return view

    def _buffer(self, name: str, rows: int, cols: int, dtype: torch.dtype, capacity_rows: Optional[int]) -> torch.Tensor:
        cap = max(capacity_rows or self.default_rows, 1)
        key = f"{name}:{cols}:{dtype}"
        buf = self._buffers.get(key)
        if buf is None or buf.shape[0] < max(rows, 1):
            if self.frozen:
                raise RuntimeError(f"workspace {key!r} must exist before graph capture")
            cap = max(cap, rows)
            if buf is not None:
                self._retired.append(buf)
                self._views.clear()              # views of the replaced buffer must not be handed out again
            buf = torch.empty((cap, cols), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:rows]

    def flat(self, name: str, numel: int, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """A 1-D buffer; with `zero` it is cleared when created (not on later calls)."""
        key = f"{name}:flat:{dtype}"
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < numel:
            if self.frozen:
                raise RuntimeError(f"workspace {key!r} must exist (and be large enough) before graph capture")
            if buf is not None:
                self._retired.append(buf)
            buf = (torch.zeros if zero else torch.empty)((max(numel, 1),), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:numel]

    def bytes_held(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


class StepMetaBuilder:
    """Collects the int32 / float32 arrays of one step and packs them into one buffer."""

    ALIGN = 4  # words: every array starts on a 16-byte boundary

    def __init__(self, q_lens: Sequence[int] = (), starts: Sequence[int] = (), pure_decode: bool = False,
                 page_size: int = 0, token_bound: int = 0):
        self.names: List[str] = []
        self.arrays: Dict[str, np.ndarray] = {}
        # the batch, for parts that derive arrays of their own from it
        self.q_lens = list(q_lens)
        self.starts = list(starts)
        self.n_seqs = len(self.q_lens)
        self.n_tokens = sum(self.q_lens)
        self.pure_decode = pure_decode
        self.page_size = page_size
        # > 0: the step is laid out for replay with this many token rows (rows beyond `n_tokens` belong to no
        # sequence, and `q_lens` ends in sequences of length 0): a part's arrays must then have sizes that follow
        # from (token_bound, n_seqs) alone, whatever the lengths are
        self.token_bound = token_bound

    def add(self, name: str, values, dtype=np.int32) -> None:
        if name in self.arrays:
            return
        arr = np.ascontiguousarray(values, dtype=dtype)
        if arr.dtype.itemsize != 4:
            raise ValueError("step metadata arrays hold 4-byte items")
        self.names.append(name)
        self.arrays[name] = arr.reshape(-1)

    def has(self, name: str) -> bool:
        return name in self.arrays

    def layout(self) -> Tuple[Dict[str, Tuple[int, int, np.dtype]], int]:
        offsets = {}
        cursor = 0
        for n in self.names:
            a = self.arrays[n]
            offsets[n] = (cursor, a.size, a.dtype)
            cursor += (a.size + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        return offsets, cursor

    def pack_into(self, host: torch.Tensor) -> Tuple[Dict[str, Tuple[int, int, np.dtype]], int]:
        """Write all arrays into the pinned int32 tensor `host`; returns (layout, words used)."""
        offsets, total = self.layout()
        if total > host.numel():
            raise RuntimeError(f"step metadata needs {total} words, the buffer holds {host.numel()}")
        view = host.numpy()
        for n, (off, size, dt) in offsets.items():
            if size:
                view[off:off + size] = self.arrays[n].view(np.int32)
        return offsets, total


@dataclass
class GroupView:
    """Device views of one cache group's per-step arrays."""
    slots: torch.Tensor          # int32 [T]: where this step's tokens are written (-1: nowhere)
    block_tables: torch.Tensor   # int32 [S * max_blocks]
    max_blocks: int


@dataclass
class StepContext:
    n_tokens: int
    n_seqs: int
    dtype: torch.dtype
    device: object
    workspace: Workspace
    # host view of the batch
    requests: List[Hashable]
    starts: List[int]
    q_lens: List[int]
    pure_decode: bool
    max_ctx: int                 # largest key count of any sequence after this step
    max_ctx_bound: int           # bound to use when launch shapes must not depend on the data
    # device views (int32 unless said otherwise)
    ids: torch.Tensor = None
    ids_from: torch.Tensor = None        # per token: row of `prev_sampled` that holds its id, or -1 (use `ids`); may be None
    prev_sampled: torch.Tensor = None    # the ids that the step before sampled, still on the device
    positions: torch.Tensor = None
    cu_q: torch.Tensor = None
    ctx_len: torch.Tensor = None
    state_slots: torch.Tensor = None
    seq_of_token: torch.Tensor = None
    groups: List[GroupView] = field(default_factory=list)
    extra: Dict[str, torch.Tensor] = field(default_factory=dict)
    fixed_shapes: bool = False   # True inside graph capture/replay: choose launch shapes from bounds
    max_seqs_bound: int = 0      # most sequences any step of this engine has

    def array(self, name: str) -> torch.Tensor:
        return self.extra[name]

    def has_array(self, name: str) -> bool:
        return name in self.extra
