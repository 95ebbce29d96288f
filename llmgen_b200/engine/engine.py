"""The serving loop: requests in, tokens out (src/runner/engine.zig:17-182).

    engine.add_request(prompt_ids, params) -> Request
    engine.step()                          -> number of requests that finished
    engine.is_finished()
    engine.last_emitted                    -> [(request, token)] of the last step

`step` = scheduler.schedule() -> executor.step(entries, sample=True) ->
scheduler.postprocess().  An empty schedule with work left is an error
(`SchedulerStuck`, src/runner/engine.zig:117-119).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import List, Sequence, Tuple

from ..sampling.params import SamplingParams
from .executor import Executor, StepEntry
from .scheduler import FINISHED, PREFILL_FIRST, BatchScheduler, Request, Scheduled, SchedulerConfig, SchedulerError


class EngineError(RuntimeError):
    pass


@dataclass
class EngineStats:
    """Counters per run (src/runner/stats.zig:15-43)."""
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    schedule_seconds: float = 0.0
    execute_seconds: float = 0.0


class Engine:
    def __init__(self, executor: Executor, config: SchedulerConfig):
        self.executor = executor
        config.max_num_seqs = min(config.max_num_seqs, executor.limits.max_num_seqs)
        if config.policy == PREFILL_FIRST and config.max_num_batched_tokens < executor.limits.max_model_len:
            # whole prompts only: a preempted sequence is computed again in one portion, so the
            # token budget must admit the longest sequence or it could never come back
            raise EngineError(f"policy prefill_first needs max_batched_tokens ({config.max_num_batched_tokens}) "
                              f">= max_model_len ({executor.limits.max_model_len}); use --policy chunked "
                              f"for a smaller budget")
        self.scheduler = BatchScheduler(executor, config)
        self.requests: List[Request] = []
        self.next_id = 0
        self.last_scheduled: List[Scheduled] = []
        self.last_emitted: List[Tuple[Request, int]] = []
        self.stats = EngineStats()

    def add_request(self, prompt: Sequence[int], params: SamplingParams = None) -> Request:
        params = params or SamplingParams()
        prompt = [int(t) for t in prompt]
        if not prompt or params.max_tokens <= 0:
            raise EngineError("empty request: a prompt and max_tokens > 0 are required")
        if len(prompt) + params.max_tokens > self.executor.limits.max_model_len:
            raise EngineError(f"sequence too long: {len(prompt)} prompt + {params.max_tokens} new tokens exceed "
                              f"max_model_len {self.executor.limits.max_model_len}")
        vocab = self.executor.model.spec.vocab_size
        for t in prompt:
            if not 0 <= t < vocab:
                raise EngineError(f"token id {t} outside the vocabulary [0, {vocab})")
        request = Request(self.next_id, prompt, params)
        request.arrival_time = time.perf_counter()
        self.next_id += 1
        self.scheduler.add(request)
        self.requests.append(request)
        return request

    def step(self) -> int:
        t0 = time.perf_counter()
        scheduled = self.scheduler.schedule()
        t1 = time.perf_counter()
        self.last_scheduled = scheduled
        if not scheduled:
            raise EngineError("scheduler stuck: work is left but nothing can be scheduled "
                              "(a request needs more pages than the pool holds)")
        entries = []
        for item in scheduled:
            r = item.request
            if r.scheduled_time == 0.0:
                r.scheduled_time = t1
            tokens = r.token_ids[item.q_start:item.q_start + item.q_len]
            entries.append(StepEntry(r.id, tokens, item.q_start, [item.q_len - 1] if item.emits() else [],
                                     r.params.temperature))
        out = self.executor.step(entries, sample=True, return_logits=False)
        t2 = time.perf_counter()
        self.last_emitted = []
        k = 0
        for item in scheduled:
            if item.emits():
                r = item.request
                if r.first_token_time == 0.0:
                    r.first_token_time = t2
                r.token_times.append(t2)
                self.last_emitted.append((r, out.token_ids[k]))
                k += 1
            if item.q_len > 1 or not item.emits():
                self.stats.prefill_tokens += item.q_len
            else:
                self.stats.decode_tokens += 1
        finished = self.scheduler.postprocess(scheduled, out.token_ids)
        for item in scheduled:
            if item.request.status == FINISHED and item.request.finish_time == 0.0:
                item.request.finish_time = t2
        self.stats.steps += 1
        self.stats.schedule_seconds += t1 - t0
        self.stats.execute_seconds += t2 - t1
        return finished

    def is_finished(self) -> bool:
        return self.scheduler.is_finished()

    def run_until_done(self) -> None:
        while not self.is_finished():
            self.step()

    def release_finished(self) -> None:
        self.requests = [r for r in self.requests if r.status != FINISHED]
        self.last_scheduled = []
        self.last_emitted = []

    def shutdown(self) -> None:
        """Give back what unfinished requests still hold (src/runner/engine.zig:74-84)."""
        for r in self.requests:
            self.executor.release(r.id)
