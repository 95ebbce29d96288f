"""The cache manager: pages of keys and values with a block table per request, one page
pool per group of layers with the same need, and slots for fixed-size per-request state.

Host-side bookkeeping only; the device arrays live in `cache/storage.py`.  The bookkeeping itself
is C++ (`csrc/runtime.cu`); the classes here are its Python face: they own the native objects,
translate request names and turn error codes into `CacheError`.

What the reference has (src/runner/block.zig:5-80): one pool for all layers, a LIFO free
stack initialised so that pops yield 0, 1, 2, ..., `ensure` / `canEnsure` / `deallocate`, and a
block table that only grows (src/runner/batching.zig:29, slot = table[pos / bs] * bs + pos % bs,
src/runner/batching.zig:74-77).  Kept: the stack order (deterministic ids), all-or-nothing
`ensure`, the dry run, freeing in reverse order, reuse without clearing.

Added here:
  * groups.  Layers that need all keys and layers that need only a window of them get page
    pools and block tables of their own.  A window group gives pages back as soon as every
    position on them is older than the window of the next token to be computed; the table keeps
    its index space (entry = -1 for a page given back), so `position // page_size` still finds
    the page of a live position.
  * state slots.  A request holds one slot index from admission to its end; layers with
    fixed-size state index their per-request arrays with it.  The pool exists even when no
    layer uses it.

Requests are named by any hashable; the native side knows them as 64-bit integers: a small
non-negative int is its own key, anything else gets a key for as long as it holds something.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong, c_void_p
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

FULL = "full"
WINDOW = "window"
_KIND_CODE = {FULL: 0, WINDOW: 1}
_FOREIGN_KEY_BASE = 1 << 62


class CacheError(RuntimeError):
    pass


_lib = None


def runtime():
    """The native runtime library (built on first use)."""
    global _lib
    if _lib is None:
        from ..kernels import build
        lib = build.load("runtime")
        for name in ("llmr_pool_new", "llmr_group_new", "llmr_group_pool", "llmr_slots_new", "llmr_cache_new",
                     "llmr_cache_group", "llmr_cache_slots", "llmr_sched_new"):
            getattr(lib, name).restype = c_void_p
        lib.llmr_group_stamp.restype = c_longlong
        lib.llmr_last_error.restype = ctypes.c_char_p
        _lib = lib
    return _lib


def _error() -> str:
    return runtime().llmr_last_error().decode("utf-8", "replace")


class RequestKeys:
    """Hashable request names -> the 64-bit keys the native side uses."""

    def __init__(self):
        self._keys: Dict[Hashable, int] = {}
        self._next = _FOREIGN_KEY_BASE

    def key(self, req: Hashable, create: bool = True) -> Optional[int]:
        if type(req) is int and 0 <= req < _FOREIGN_KEY_BASE:
            return req
        k = self._keys.get(req)
        if k is None and create:
            k = self._next
            self._next += 1
            self._keys[req] = k
        return k

    def forget(self, req: Hashable) -> None:
        self._keys.pop(req, None)


def _ints(n: int):
    return (c_int * max(n, 1))()


class PagePool:
    """A stack of free page ids; a fresh pool hands out 0, 1, 2, ..."""

    def __init__(self, num_pages: int, _handle=None):
        if num_pages < 0:
            raise CacheError(f"a page pool cannot hold {num_pages} pages")
        self.num_pages = num_pages
        self._owned = _handle is None
        self._h = c_void_p(_handle) if _handle is not None else c_void_p(runtime().llmr_pool_new(c_int(num_pages)))

    def __del__(self):
        if getattr(self, "_owned", False) and _lib is not None and self._h:
            _lib.llmr_pool_delete(self._h)
            self._h = None

    @property
    def num_free(self) -> int:
        return int(runtime().llmr_pool_num_free(self._h))

    def take(self, n: int) -> Optional[List[int]]:
        """n pages, or None (and no change) if fewer are free."""
        out = _ints(n)
        if not runtime().llmr_pool_take(self._h, c_int(n), out):
            return None
        return list(out[:n])

    def give(self, pages: Sequence[int]) -> None:
        arr = (c_int * max(len(pages), 1))(*pages)
        if runtime().llmr_pool_give(self._h, arr, c_int(len(pages))) != 0:
            raise CacheError(_error())

    def free_list(self) -> List[int]:
        out = _ints(self.num_pages)
        n = runtime().llmr_pool_free_list(self._h, out, c_int(self.num_pages))
        return list(out[:n])


@dataclass(frozen=True)
class GroupSpec:
    """One kind of need: every key (`FULL`) or the last `window` keys (`WINDOW`)."""
    kind: str
    window: int = 0

    def __post_init__(self):
        if self.kind not in (FULL, WINDOW):
            raise CacheError(f"unknown cache group kind {self.kind!r}")
        if self.kind == WINDOW and self.window <= 0:
            raise CacheError("a window group needs a positive window")


class CacheGroup:
    """Pages and block tables of one group of layers."""

    def __init__(self, spec: GroupSpec, num_pages: int, page_size: int, _handle=None, _keys: Optional[RequestKeys] = None):
        if page_size <= 0:
            raise CacheError(f"page size {page_size}")
        if num_pages < 0:
            raise CacheError(f"a page pool cannot hold {num_pages} pages")
        self.spec = spec
        self.page_size = page_size
        self.num_pages = num_pages
        self._keys = _keys or RequestKeys()
        self._owned = _handle is None
        lib = runtime()
        self._h = c_void_p(_handle) if _handle is not None else c_void_p(
            lib.llmr_group_new(c_int(_KIND_CODE[spec.kind]), c_int(spec.window), c_int(num_pages), c_int(page_size)))
        self.pool = PagePool(num_pages, _handle=lib.llmr_group_pool(self._h))
        self._buf = _ints(64)

    def __del__(self):
        if getattr(self, "_owned", False) and _lib is not None and self._h:
            _lib.llmr_group_delete(self._h)
            self._h = None

    # -- queries
    def table(self, req: Hashable) -> List[int]:
        k = self._keys.key(req, create=False)
        if k is None:
            return []
        n = runtime().llmr_group_table(self._h, c_longlong(k), self._buf, c_int(len(self._buf)))
        if n > len(self._buf):
            self._buf = _ints(2 * n)
            n = runtime().llmr_group_table(self._h, c_longlong(k), self._buf, c_int(len(self._buf)))
        return list(self._buf[:n]) if n > 0 else []

    def has_table(self, req: Hashable) -> bool:
        k = self._keys.key(req, create=False)
        return k is not None and runtime().llmr_group_table(self._h, c_longlong(k), self._buf, c_int(0)) >= 0

    def table_stamp(self, req: Hashable):
        """Changes whenever the contents of `req`'s table may have changed: a full-attention table
        only grows, a windowed one also loses pages, so it has no stamp (None)."""
        if self.spec.kind == WINDOW:
            return None
        k = self._keys.key(req, create=False)
        return int(runtime().llmr_group_stamp(self._h, c_longlong(k))) if k is not None else 0

    def first_needed_position(self, start: int) -> int:
        """Oldest position that the token at `start` still attends to."""
        if self.spec.kind == WINDOW:
            return max(0, start - self.spec.window + 1)
        return 0

    @property
    def num_tables(self) -> int:
        return int(runtime().llmr_group_num_tables(self._h))

    def can_reserve(self, req: Hashable, start: int, end: int) -> bool:
        return bool(runtime().llmr_group_can_reserve(self._h, c_longlong(self._keys.key(req)), c_int(start), c_int(end)))

    def reserve(self, req: Hashable, start: int, end: int) -> bool:
        """Make positions [start, end) writable for `req`; all or nothing."""
        return bool(runtime().llmr_group_reserve(self._h, c_longlong(self._keys.key(req)), c_int(start), c_int(end)))

    def release(self, req: Hashable) -> None:
        k = self._keys.key(req, create=False)
        if k is not None:
            runtime().llmr_group_release(self._h, c_longlong(k))

    def slot_of(self, req: Hashable, pos: int) -> int:
        if not self.has_table(req):
            raise KeyError(req)
        page = self.table(req)[pos // self.page_size]
        if page < 0:
            raise CacheError(f"position {pos} of request {req!r} lies on a page that was given back")
        return page * self.page_size + pos % self.page_size

    def pages_held(self, req: Hashable) -> int:
        return sum(1 for p in self.table(req) if p >= 0)

    def check(self, index: int = 0) -> None:
        if runtime().llmr_group_check(self._h, c_int(index)) != 0:
            raise CacheError(_error())


class StateSlots:
    """Indices into per-request arrays of fixed size."""

    def __init__(self, num_slots: int, _handle=None, _keys: Optional[RequestKeys] = None):
        self.num_slots = num_slots
        self._keys = _keys or RequestKeys()
        self._owned = _handle is None
        self._h = c_void_p(_handle) if _handle is not None else c_void_p(runtime().llmr_slots_new(c_int(num_slots)))

    def __del__(self):
        if getattr(self, "_owned", False) and _lib is not None and self._h:
            _lib.llmr_slots_delete(self._h)
            self._h = None

    @property
    def num_free(self) -> int:
        return int(runtime().llmr_slots_num_free(self._h))

    def take(self, req: Hashable) -> Optional[int]:
        s = int(runtime().llmr_slots_take(self._h, c_longlong(self._keys.key(req))))
        return s if s >= 0 else None

    def give(self, req: Hashable) -> None:
        k = self._keys.key(req, create=False)
        if k is not None:
            runtime().llmr_slots_give(self._h, c_longlong(k))

    def holds(self, req: Hashable) -> bool:
        k = self._keys.key(req, create=False)
        return k is not None and runtime().llmr_slots_slot(self._h, c_longlong(k)) >= 0

    def slot(self, req: Hashable) -> int:
        k = self._keys.key(req, create=False)
        s = int(runtime().llmr_slots_slot(self._h, c_longlong(k))) if k is not None else -1
        if s < 0:
            raise KeyError(req)
        return s


class FreshSlots:
    """The state slots handed out since the executor last looked (a live view of the native list)."""

    def __init__(self, cache_handle):
        self._h = cache_handle

    def _items(self, clear: bool = False) -> List[int]:
        out = _ints(256)
        n = runtime().llmr_cache_fresh(self._h, out, c_int(256), c_int(0))
        if n > 256:
            out = _ints(n)
            runtime().llmr_cache_fresh(self._h, out, c_int(n), c_int(0))
        items = list(out[:n])
        if clear:
            runtime().llmr_cache_fresh(self._h, out, c_int(0), c_int(1))
        return items

    def __iter__(self):
        return iter(self._items())

    def __len__(self) -> int:
        return len(self._items())

    def __bool__(self) -> bool:
        return runtime().llmr_cache_fresh(self._h, None, c_int(0), c_int(0)) > 0

    def __eq__(self, other) -> bool:
        return self._items() == list(other)

    def __repr__(self) -> str:
        return repr(self._items())

    def clear(self) -> None:
        self._items(clear=True)


class CacheManager:
    """All groups and the state slots; every operation is all-or-nothing over the groups."""

    def __init__(self, group_specs: Sequence[GroupSpec], pages_per_group: Sequence[int], page_size: int,
                 num_state_slots: int):
        if len(group_specs) != len(pages_per_group):
            raise CacheError("one page count per group is required")
        if page_size <= 0:
            raise CacheError(f"page size {page_size}")
        self.page_size = page_size
        lib = runtime()
        n = len(group_specs)
        kinds = (c_int * max(n, 1))(*[_KIND_CODE[s.kind] for s in group_specs])
        windows = (c_int * max(n, 1))(*[s.window for s in group_specs])
        pages = (c_int * max(n, 1))(*pages_per_group)
        self._h = c_void_p(lib.llmr_cache_new(c_int(n), kinds, windows, pages, c_int(page_size), c_int(num_state_slots)))
        if not self._h:
            raise CacheError("bad cache geometry (pages, page size and slots must not be negative)")
        self._keys = RequestKeys()
        self.groups = [CacheGroup(s, p, page_size, _handle=lib.llmr_cache_group(self._h, c_int(i)), _keys=self._keys)
                       for i, (s, p) in enumerate(zip(group_specs, pages_per_group))]
        self.state = StateSlots(num_state_slots, _handle=lib.llmr_cache_slots(self._h), _keys=self._keys)
        self.fresh_state = FreshSlots(self._h)

    def __del__(self):
        if _lib is not None and getattr(self, "_h", None):
            _lib.llmr_cache_delete(self._h)
            self._h = None

    @property
    def native_handle(self) -> c_void_p:
        return self._h

    def key(self, req: Hashable) -> int:
        """The 64-bit name under which the native side knows `req`."""
        return self._keys.key(req)

    def forget(self, req: Hashable) -> None:
        """Drop the name of a request that the native side has already released."""
        self._keys.forget(req)

    # -- admission
    def admit(self, req: Hashable) -> Optional[int]:
        """Give `req` a state slot (None when all are taken).  Idempotent."""
        s = int(runtime().llmr_cache_admit(self._h, c_longlong(self._keys.key(req))))
        return s if s >= 0 else None

    def is_admitted(self, req: Hashable) -> bool:
        return self.state.holds(req)

    # -- pages
    def can_reserve(self, req: Hashable, start: int, end: int) -> bool:
        return bool(runtime().llmr_cache_can_reserve(self._h, c_longlong(self._keys.key(req)), c_int(start), c_int(end)))

    def reserve(self, req: Hashable, start: int, end: int) -> bool:
        """Pages for computing positions [start, end) of `req` in every group, or no change."""
        return bool(runtime().llmr_cache_reserve(self._h, c_longlong(self._keys.key(req)), c_int(start), c_int(end)))

    def release(self, req: Hashable) -> None:
        """Everything `req` holds goes back: pages of every group and its state slot."""
        k = self._keys.key(req, create=False)
        if k is not None:
            runtime().llmr_cache_release(self._h, c_longlong(k))
            self._keys.forget(req)

    def release_pages(self, req: Hashable) -> None:
        """Pages only (a preempted request keeps nothing but may be admitted again)."""
        k = self._keys.key(req, create=False)
        if k is not None:
            runtime().llmr_cache_release_pages(self._h, c_longlong(k))

    def check_step(self, req: Hashable, start: int, n: int) -> Optional[str]:
        """Why a step cannot compute positions [start, start + n) of `req`, or None if it can."""
        k = self._keys.key(req, create=False)
        rc = 1 if k is None else runtime().llmr_cache_check_step(self._h, c_longlong(k), c_int(start), c_int(n))
        if rc == 0:
            return None
        if rc == 1:
            return f"request {req!r} was not admitted"
        return f"request {req!r}: no pages reserved for positions up to {start + n - 1}"

    # -- accounting, for tests and the leak check at the end of a run
    def num_free_pages(self) -> List[int]:
        return [g.pool.num_free for g in self.groups]

    def all_free(self) -> bool:
        return (all(g.pool.num_free == g.pool.num_pages and g.num_tables == 0 for g in self.groups)
                and self.state.num_free == self.state.num_slots)

    def check_consistency(self) -> None:
        """No page lost, none held twice: held + free == all, per group."""
        for gi, g in enumerate(self.groups):
            g.check(gi)
