"""Plain restatement of the host runtime, kept under tests/ as the oracle of the C++ one
(llmgen_b200/csrc/runtime.cu): the cache manager (page pools, groups, block tables, state slots)
and the batch scheduler, in straightforward Python.  Rules and citations are those of the product
files `llmgen_b200/cache/manager.py` and `llmgen_b200/engine/scheduler.py`; no code is shared with
them beyond the request / configuration records."""
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


# ------------------------------------------------------------------ scheduler
from llmgen_b200.engine.scheduler import (CHUNKED, FINISHED, PREFILL_FIRST, RUNNING, WAITING, Request, Scheduled,
                                          SchedulerConfig)


class PlainBatchScheduler:
    def __init__(self, cache, config: SchedulerConfig):
        self.cache = cache          # anything with admit / reserve / can_reserve / release
        self.config = config
        self.waiting: List[Request] = []
        self.running: List[Request] = []
        self.num_preemptions = 0

    def is_finished(self) -> bool:
        return not self.waiting and not self.running

    def add(self, request: Request) -> None:
        request.status = WAITING
        self.waiting.append(request)

    # ---------------------------------------------------------------- scheduling
    def schedule(self) -> List[Scheduled]:
        if self.config.policy == PREFILL_FIRST:
            return self._schedule_prefill_first()
        return self._schedule_chunked()

    def _admit(self, request: Request, upto: int) -> bool:
        """State slot and pages for positions [0, upto) of a waiting request, or nothing."""
        if len(self.running) >= self.config.max_num_seqs:
            return False
        admitted = self.cache.admit(request.id)     # a slot number (0 counts) or True; None / False: full
        if admitted is None or admitted is False:
            return False
        if not self.cache.reserve(request.id, 0, upto):
            self.cache.release(request.id)
            return False
        return True

    def _make_room(self, index: int, start: int, upto: int) -> bool:
        """Preempt from the tail of `running` until positions [start, upto) of running[index]
        can be reserved.  False if the sequence had to preempt itself."""
        request = self.running[index]
        while not self.cache.can_reserve(request.id, start, upto):
            if len(self.running) - 1 > index:
                self._preempt(self.running.pop())
            else:
                self.running.pop(index)
                self._preempt(request)
                return False
        return True

    def _schedule_prefill_first(self) -> List[Scheduled]:
        cfg = self.config
        out: List[Scheduled] = []
        tokens = 0
        while self.waiting and len(out) < cfg.max_num_seqs:
            request = self.waiting[0]
            n = len(request)
            if tokens + n > cfg.max_num_batched_tokens:
                break
            if not self._admit(request, n):
                break
            self.waiting.pop(0)
            request.status = RUNNING
            request.num_computed_tokens = 0
            self.running.append(request)
            out.append(Scheduled(request, 0, n))
            tokens += n
        if out:
            return out
        i = 0
        while i < len(self.running) and len(out) < cfg.max_num_seqs:
            request = self.running[i]
            n = len(request)
            if not self._make_room(i, n - 1, n):
                break
            ok = self.cache.reserve(request.id, n - 1, n)
            assert ok
            out.append(Scheduled(request, n - 1, 1))
            i += 1
        return out

    def _schedule_chunked(self) -> List[Scheduled]:
        cfg = self.config
        out: List[Scheduled] = []
        budget = cfg.max_num_batched_tokens
        prefill_budget = cfg.chunk_tokens
        preemptions_before = self.num_preemptions
        i = 0
        while i < len(self.running) and len(out) < cfg.max_num_seqs and budget > 0:
            request = self.running[i]
            remaining = len(request) - request.num_computed_tokens
            in_prefill = remaining > 1
            q_len = min(remaining, budget)
            if in_prefill:
                q_len = min(q_len, prefill_budget)
            if q_len == 0:
                i += 1
                continue
            start = request.num_computed_tokens
            if not self._make_room(i, start, start + q_len):
                break
            ok = self.cache.reserve(request.id, start, start + q_len)
            assert ok
            out.append(Scheduled(request, start, q_len))
            budget -= q_len
            if in_prefill:
                prefill_budget -= q_len
            i += 1
        if self.num_preemptions != preemptions_before:
            return out
        while self.waiting and len(out) < cfg.max_num_seqs and budget > 0 and prefill_budget > 0:
            request = self.waiting[0]
            q_len = min(len(request), budget, prefill_budget)
            if not self._admit(request, q_len):
                break
            self.waiting.pop(0)
            request.status = RUNNING
            request.num_computed_tokens = 0
            self.running.append(request)
            out.append(Scheduled(request, 0, q_len))
            budget -= q_len
            prefill_budget -= q_len
        return out

    def _preempt(self, request: Request) -> None:
        request.status = WAITING
        request.num_computed_tokens = 0
        request.num_preemptions += 1
        self.cache.release(request.id)
        self.waiting.insert(0, request)
        self.num_preemptions += 1

    # ---------------------------------------------------------------- after the step
    def postprocess(self, scheduled: Sequence[Scheduled], tokens: Sequence[int]) -> int:
        """Record what the step computed; append the new token of every emitting portion
        (`tokens`, in order); finish on EOS or max_tokens and free (src/runner/batching.zig:323-355).
        Returns the number of requests that finished."""
        k = 0
        finished = 0
        for item in scheduled:
            request = item.request
            emits = item.emits()
            request.num_computed_tokens = item.q_start + item.q_len
            if not emits:
                continue
            token = int(tokens[k])
            k += 1
            request.token_ids.append(token)
            hit_eos = (not request.params.ignore_eos) and token in self.config.eos_token_ids
            if hit_eos or request.num_completion_tokens >= request.params.max_tokens:
                request.status = FINISHED
                self.cache.release(request.id)
                if request in self.running:
                    self.running.remove(request)
                finished += 1
        return finished
