"""The batch scheduler: admits requests, cuts prompts into portions under a token budget,
decodes, finishes and frees, and decides what happens when pages run out.

Policies and rules are the reference's (src/runner/batching.zig:111-356):

  prefill_first  admit whole prompts from the head of `waiting` while sequences, the token
                 budget and pages allow; a step that admitted anything is prefill-only;
                 otherwise one decode token for each running sequence in order.
  chunked        first serve `running` in order (decode rows cost 1, unfinished prompts take
                 min(remaining, token budget, prefill budget)), then, only if nothing was
                 preempted this round, admit from `waiting` with pages for just that portion.

When pages run out for the sequence being scheduled, the LAST running sequence is preempted
(its pages and state slot go back, it returns to the FRONT of `waiting` and is later computed
again from position 0, generated tokens included); if the sequence is itself the last, it
preempts itself and scheduling stops for this step.

The decisions are taken in C++ (`csrc/runtime.cu`, next to the cache manager whose pages they
spend); `BatchScheduler` here owns the native scheduler, hands requests to it and mirrors what it
decided into the `Request` objects.  Pure host logic, so it is tested without a GPU.
"""
from __future__ import annotations

from ctypes import byref, c_int, c_longlong, c_void_p
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

from ..cache.manager import CacheManager, runtime
from ..sampling.params import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"
PREFILL_FIRST, CHUNKED = "prefill_first", "chunked"


class SchedulerError(RuntimeError):
    pass


class Request:
    """One sequence: prompt and generated ids, and how much of it is in the cache
    (src/runner/batching.zig:18-78)."""

    def __init__(self, req_id: int, prompt: Sequence[int], params: SamplingParams):
        self.id = req_id
        self.token_ids: List[int] = list(prompt)
        self.num_prompt_tokens = len(self.token_ids)
        self.num_computed_tokens = 0
        self.params = params
        self.status = WAITING
        self.num_preemptions = 0
        self.arrival_time = 0.0
        self.scheduled_time = 0.0
        self.first_token_time = 0.0
        self.finish_time = 0.0
        self.token_times: List[float] = []

    def __len__(self) -> int:
        return len(self.token_ids)

    @property
    def num_completion_tokens(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def completion(self) -> List[int]:
        return self.token_ids[self.num_prompt_tokens:]


@dataclass
class Scheduled:
    """`q_len` tokens of `request` starting at `q_start` (src/runner/batching.zig:92-103)."""
    request: Request
    q_start: int
    q_len: int
    emit: Optional[bool] = None      # set by the scheduler; None: decided from the request's length

    def emits(self) -> bool:
        """True when the portion reaches the last token of the sequence, so the step yields a new one.
        The scheduler says so itself: a token of the step before may not have been read yet, and the
        request's list is then one short."""
        if self.emit is not None:
            return self.emit
        return self.q_start + self.q_len == len(self.request)


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 16384
    policy: str = PREFILL_FIRST
    chunk_tokens: int = 2048
    eos_token_ids: Sequence[int] = ()

    def __post_init__(self):
        if self.policy not in (PREFILL_FIRST, CHUNKED):
            raise SchedulerError(f"unknown policy {self.policy!r} (prefill_first | chunked)")


class BatchScheduler:
    """The native scheduler and its Python mirror.

    `cache` is the `CacheManager` whose pages are spent, or anything that holds it as `.cache`
    (the executor).  State slots that admissions hand out are listed by the manager
    (`fresh_state`); whoever owns per-request state clears them before the next step."""

    _POLICY_CODE = {PREFILL_FIRST: 0, CHUNKED: 1}
    _STATUS = {0: WAITING, 1: RUNNING, 2: FINISHED}

    def __init__(self, cache, config: SchedulerConfig):
        manager = cache if isinstance(cache, CacheManager) else getattr(cache, "cache", None)
        if not isinstance(manager, CacheManager):
            raise SchedulerError("the scheduler needs a CacheManager (or an executor that holds one as .cache)")
        self.cache = cache
        self.manager = manager
        self.config = config
        self._lib = runtime()
        eos = [int(t) for t in config.eos_token_ids]
        self._eos_sent = tuple(eos)
        self._h = c_void_p(self._lib.llmr_sched_new(
            manager.native_handle, c_int(self._POLICY_CODE[config.policy]), c_int(config.max_num_seqs),
            c_int(config.max_num_batched_tokens), c_int(config.chunk_tokens), (c_int * max(len(eos), 1))(*eos),
            c_int(len(eos))))
        if not self._h:
            raise SchedulerError("the native scheduler refused its configuration")
        self._requests: Dict[int, Request] = {}       # native key -> request, while the scheduler knows it
        self._cap = 0
        self._grow(max(16, min(config.max_num_seqs, 4096)))

    def __del__(self):
        if getattr(self, "_h", None) and self._lib is not None:
            self._lib.llmr_sched_delete(self._h)
            self._h = None

    def _grow(self, cap: int) -> None:
        self._cap = cap
        self._keys = (c_longlong * cap)()
        self._starts = (c_int * cap)()
        self._lens = (c_int * cap)()
        self._tokens = (c_int * cap)()
        self._flags = (c_int * cap)()
        self._other = (c_longlong * cap)()
        self._count = c_int(0)

    # ---------------------------------------------------------------- queues
    def _queue(self, which: int) -> List[Request]:
        n = self._lib.llmr_sched_queue(self._h, c_int(which), self._other, c_int(self._cap))
        if n > self._cap:
            self._grow(2 * n)
            n = self._lib.llmr_sched_queue(self._h, c_int(which), self._other, c_int(self._cap))
        return [self._requests[self._other[i]] for i in range(n)]

    @property
    def waiting(self) -> List[Request]:
        return self._queue(0)

    @property
    def running(self) -> List[Request]:
        return self._queue(1)

    @property
    def num_preemptions(self) -> int:
        return int(self._lib.llmr_sched_num_preemptions(self._h))

    def is_finished(self) -> bool:
        return bool(self._lib.llmr_sched_is_finished(self._h))

    def add(self, request: Request) -> None:
        if len(request) != request.num_prompt_tokens:
            raise SchedulerError("a request is added before it has generated tokens")
        key = self.manager.key(request.id)
        if key in self._requests:
            raise SchedulerError(f"request {request.id!r} is already scheduled")
        request.status = WAITING
        self._requests[key] = request
        if len(self._requests) > self._cap:
            self._grow(2 * self._cap)
        self._lib.llmr_sched_add(self._h, c_longlong(key), c_int(len(request)), c_int(request.params.max_tokens),
                                 c_int(1 if request.params.ignore_eos else 0))

    # ---------------------------------------------------------------- scheduling
    def schedule(self) -> List[Scheduled]:
        """This step's portions.  Requests that lost their place are back at the front of `waiting`
        with nothing computed."""
        n = self._lib.llmr_sched_schedule(self._h, self._keys, self._starts, self._lens, self._flags, c_int(self._cap),
                                          self._other, c_int(self._cap), byref(self._count))
        assert n <= self._cap and self._count.value <= self._cap     # both are bounded by the known requests
        for i in range(self._count.value):
            request = self._requests[self._other[i]]
            request.status = WAITING
            request.num_computed_tokens = 0
            request.num_preemptions += 1
        out = []
        for i in range(n):
            request = self._requests[self._keys[i]]
            request.status = RUNNING
            if self._starts[i] == 0:
                request.num_computed_tokens = 0
            out.append(Scheduled(request, self._starts[i], self._lens[i], bool(self._flags[i])))
        return out

    # ---------------------------------------------------------------- after the step
    def _sync_eos(self) -> None:
        if tuple(self.config.eos_token_ids) != self._eos_sent:       # the configuration's list is the one that counts
            self._eos_sent = tuple(int(t) for t in self.config.eos_token_ids)
            self._lib.llmr_sched_set_eos(self._h, (c_int * max(len(self._eos_sent), 1))(*self._eos_sent),
                                         c_int(len(self._eos_sent)))

    def advance(self, scheduled: Sequence[Scheduled]) -> None:
        """Once a step has been launched: record what it computes and let every sequence whose portion
        reached its end grow by the token to come; a request that has its max_tokens with that token
        leaves the queues now and frees what it holds (the step may still be running: what it frees
        is written again only by later steps, which the GPU runs after this one).  The tokens
        themselves come with `resolve`."""
        n = len(scheduled)
        if n > self._cap:
            self._grow(2 * n)
        for i, item in enumerate(scheduled):
            self._keys[i] = self.manager.key(item.request.id)
            self._starts[i] = item.q_start
            self._lens[i] = item.q_len
            if item.request.status != FINISHED:
                item.request.num_computed_tokens = item.q_start + item.q_len
        self._lib.llmr_sched_advance(self._h, c_int(n), self._keys, self._starts, self._lens)

    def resolve(self, scheduled: Sequence[Scheduled], tokens: Sequence[int]) -> int:
        """The tokens of a step that `advance` has recorded, in the order of its emitting portions:
        appended to their requests; a request whose sequence the token ends (EOS, unless ignored) or
        whose max_tokens it fills is finished and freed (src/runner/batching.zig:323-355).  A token
        sampled for a request that had already ended (the step was launched before that was known)
        is dropped.  Returns the number of requests that finished."""
        self._sync_eos()
        emitting = [item for item in scheduled if item.emits()]
        n = len(emitting)
        if n > self._cap:
            self._grow(2 * n)
        for i, item in enumerate(emitting):
            self._keys[i] = self.manager.key(item.request.id)
            self._tokens[i] = int(tokens[i])
        done = self._lib.llmr_sched_resolve(self._h, c_int(n), self._keys, self._tokens, self._flags)
        for i, item in enumerate(emitting):
            last = self._flags[i]
            if last < 0:
                continue
            request = item.request
            request.token_ids.append(int(tokens[i]))
            if last == 1:
                request.status = FINISHED
                self._requests.pop(self._keys[i], None)
                self.manager.forget(request.id)
        return done

    def postprocess(self, scheduled: Sequence[Scheduled], tokens: Sequence[int]) -> int:
        """`advance` and `resolve` in one: for steps whose tokens are read before the next one is
        scheduled."""
        self.advance(scheduled)
        return self.resolve(scheduled, tokens)
