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

Pure host logic over the cache manager's interface (`admit`, `reserve`, `can_reserve`,
`release`), so it is tested without a GPU.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

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

    def emits(self) -> bool:
        """True when the portion reaches the last known token, so the step yields a new one."""
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
