"""The cache manager: pages of keys and values with a block table per request, one page
pool per group of layers with the same need, and slots for fixed-size per-request state.

Host-side bookkeeping only; the device arrays live in `cache/storage.py`.

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
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

FULL = "full"
WINDOW = "window"


class CacheError(RuntimeError):
    pass


class PagePool:
    """A stack of free page ids; a fresh pool hands out 0, 1, 2, ..."""

    def __init__(self, num_pages: int):
        if num_pages < 0:
            raise CacheError(f"a page pool cannot hold {num_pages} pages")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._is_free = [True] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self, n: int) -> Optional[List[int]]:
        """n pages, or None (and no change) if fewer are free."""
        if n > len(self._free):
            return None
        out = []
        for _ in range(n):
            p = self._free.pop()
            self._is_free[p] = False
            out.append(p)
        return out

    def give(self, pages: Sequence[int]) -> None:
        for p in pages:
            if p < 0 or p >= self.num_pages:
                raise CacheError(f"page {p} does not belong to this pool of {self.num_pages}")
            if self._is_free[p]:
                raise CacheError(f"page {p} freed twice")
            self._is_free[p] = True
            self._free.append(p)


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

    def __init__(self, spec: GroupSpec, num_pages: int, page_size: int):
        if page_size <= 0:
            raise CacheError(f"page size {page_size}")
        self.spec = spec
        self.page_size = page_size
        self.pool = PagePool(num_pages)
        self.tables: Dict[Hashable, List[int]] = {}
        self.births: Dict[Hashable, int] = {}      # which table of the group's history a request's table is
        self._born = 0

    # -- queries
    def table(self, req: Hashable) -> List[int]:
        return self.tables.get(req, [])

    def table_stamp(self, req: Hashable):
        """Changes whenever the contents of `req`'s table may have changed: a full-attention table
        only grows, a windowed one also loses pages, so its stamp is never equal to an earlier one."""
        if self.spec.kind == WINDOW:
            return None
        return (self.births.get(req, 0), len(self.tables.get(req, ())))

    def first_needed_position(self, start: int) -> int:
        """Oldest position that the token at `start` still attends to."""
        if self.spec.kind == WINDOW:
            return max(0, start - self.spec.window + 1)
        return 0

    def _plan(self, req: Hashable, start: int, end: int):
        """(pages to give back, number of new pages) for computing positions [start, end)."""
        table = self.tables.get(req, [])
        ps = self.page_size
        first_live_page = self.first_needed_position(start) // ps
        give = [i for i in range(min(first_live_page, len(table))) if table[i] >= 0]
        need_pages = (end + ps - 1) // ps
        new = max(0, need_pages - len(table))
        # positions between the end of the table and the first live page need no real page
        skipped = max(0, min(first_live_page, need_pages) - len(table))
        return give, new - skipped, skipped

    def can_reserve(self, req: Hashable, start: int, end: int) -> bool:
        give, new, _ = self._plan(req, start, end)
        return new <= self.pool.num_free + len(give)

    def reserve(self, req: Hashable, start: int, end: int) -> bool:
        """Make positions [start, end) writable for `req`; all or nothing."""
        give, new, skipped = self._plan(req, start, end)
        if new > self.pool.num_free + len(give):
            return False
        table = self.tables.get(req)
        if table is None:
            table = self.tables[req] = []
            self._born += 1
            self.births[req] = self._born
        self.pool.give([table[i] for i in give])
        for i in give:
            table[i] = -1
        table.extend([-1] * skipped)
        pages = self.pool.take(new)
        assert pages is not None
        table.extend(pages)
        return True

    def release(self, req: Hashable) -> None:
        table = self.tables.pop(req, None)
        self.births.pop(req, None)
        if table:
            self.pool.give([p for p in reversed(table) if p >= 0])

    def slot_of(self, req: Hashable, pos: int) -> int:
        page = self.tables[req][pos // self.page_size]
        if page < 0:
            raise CacheError(f"position {pos} of request {req!r} lies on a page that was given back")
        return page * self.page_size + pos % self.page_size

    def pages_held(self, req: Hashable) -> int:
        return sum(1 for p in self.tables.get(req, []) if p >= 0)


class StateSlots:
    """Indices into per-request arrays of fixed size."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self.owner: Dict[Hashable, int] = {}

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self, req: Hashable) -> Optional[int]:
        if req in self.owner:
            return self.owner[req]
        if not self._free:
            return None
        s = self._free.pop()
        self.owner[req] = s
        return s

    def give(self, req: Hashable) -> None:
        s = self.owner.pop(req, None)
        if s is not None:
            self._free.append(s)

    def slot(self, req: Hashable) -> int:
        return self.owner[req]


class CacheManager:
    """All groups and the state slots; every operation is all-or-nothing over the groups."""

    def __init__(self, group_specs: Sequence[GroupSpec], pages_per_group: Sequence[int], page_size: int,
                 num_state_slots: int):
        if len(group_specs) != len(pages_per_group):
            raise CacheError("one page count per group is required")
        self.page_size = page_size
        self.groups = [CacheGroup(s, n, page_size) for s, n in zip(group_specs, pages_per_group)]
        self.state = StateSlots(num_state_slots)
        self.fresh_state: List[int] = []   # slots handed out since the executor last looked

    # -- admission
    def admit(self, req: Hashable) -> Optional[int]:
        """Give `req` a state slot (None when all are taken).  Idempotent."""
        known = req in self.state.owner
        slot = self.state.take(req)
        if slot is not None and not known:
            self.fresh_state.append(slot)
        return slot

    def is_admitted(self, req: Hashable) -> bool:
        return req in self.state.owner

    # -- pages
    def can_reserve(self, req: Hashable, start: int, end: int) -> bool:
        return all(g.can_reserve(req, start, end) for g in self.groups)

    def reserve(self, req: Hashable, start: int, end: int) -> bool:
        """Pages for computing positions [start, end) of `req` in every group, or no change."""
        if not self.can_reserve(req, start, end):
            return False
        for g in self.groups:
            ok = g.reserve(req, start, end)
            assert ok
        return True

    def release(self, req: Hashable) -> None:
        """Everything `req` holds goes back: pages of every group and its state slot."""
        for g in self.groups:
            g.release(req)
        self.state.give(req)

    def release_pages(self, req: Hashable) -> None:
        """Pages only (a preempted request keeps nothing but may be admitted again)."""
        for g in self.groups:
            g.release(req)

    # -- accounting, for tests and the leak check at the end of a run
    def num_free_pages(self) -> List[int]:
        return [g.pool.num_free for g in self.groups]

    def all_free(self) -> bool:
        return (all(g.pool.num_free == g.pool.num_pages and not g.tables for g in self.groups)
                and self.state.num_free == self.state.num_slots)

    def check_consistency(self) -> None:
        """No page lost, none held twice: held + free == all, per group."""
        for gi, g in enumerate(self.groups):
            held = [p for t in g.tables.values() for p in t if p >= 0]
            if len(held) != len(set(held)):
                raise CacheError(f"group {gi}: a page is held twice")
            free = list(g.pool._free)
            if len(free) != len(set(free)):
                raise CacheError(f"group {gi}: a page is on the free stack twice")
            if set(held) & set(free):
                raise CacheError(f"group {gi}: a page is both held and free")
            if len(held) + len(free) != g.pool.num_pages:
                raise CacheError(f"group {gi}: {g.pool.num_pages - len(held) - len(free)} page(s) lost")
