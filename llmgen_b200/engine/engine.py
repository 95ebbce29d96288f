"""The serving loop: requests in, tokens out (src/runner/engine.zig:17-182).

    engine.add_request(prompt_ids, params) -> Request
    engine.step()                          -> number of requests that finished
    engine.is_finished()
    engine.last_emitted                    -> [(request, token)] of the last step

`step` = scheduler.schedule() -> executor.step(entries, sample=True) ->
scheduler.advance() + resolve().  An empty schedule with work left is an error
(`SchedulerStuck`, src/runner/engine.zig:117-119).

Decode steps run one ahead of the host (`Engine.run_ahead`, on by default): step k+1 is scheduled
and launched while step k runs, with its ids taken on the device from step k's sampler, and only
then are step k's ids read.  The reference reads every step's ids before it schedules the next
(src/runner/engine.zig:121-160); there the GPU idles while the host schedules, fills the step's
arrays and launches the graph.
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
        self.run_ahead = True        # launch decode steps before the tokens of the step before are read
        self._inflight = None        # (schedule, pending ids, request -> row) of a launched step not yet read

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
        """Schedule and launch one step; returns how many requests finished with the tokens that
        became known in this call (`last_emitted`).

        Steps of single decoded tokens replayed from a graph run one ahead: the step is launched with
        its input ids taken on the device from what the step before sampled, and only then are that
        earlier step's ids read, so the host's work for a step overlaps the GPU's work on it.  The
        tokens named by a call are then those of the step launched by the call before.  A request
        that turns out to have ended (an end-of-sequence token) may have been given one more row in
        the step already launched; that row's token is dropped.  Any other kind of step (prompts,
        portions, eager mode) first reads what is still in flight and is itself read at once."""
        t0 = time.perf_counter()
        scheduled = self.scheduler.schedule()
        t1 = time.perf_counter()
        if not scheduled:
            if self._inflight is not None:
                return self._read_inflight()
            raise EngineError("scheduler stuck: work is left but nothing can be scheduled "
                              "(a request needs more pages than the pool holds)")
        ahead = self.run_ahead and not self.executor.eager and all(x.q_len == 1 and x.emits() for x in scheduled)
        finished = 0
        emitted_before: List[Tuple[Request, int]] = []
        if not ahead and self._inflight is not None:
            finished = self._read_inflight()
            emitted_before = self.last_emitted
            scheduled = [x for x in scheduled if x.request.status != FINISHED]     # an end-of-sequence token came in
            if not scheduled:
                return finished
        for item in scheduled:
            if item.request.scheduled_time == 0.0:
                item.request.scheduled_time = t1
            if item.q_len > 1 or not item.emits():
                self.stats.prefill_tokens += item.q_len
            else:
                self.stats.decode_tokens += 1
        self.stats.steps += 1
        self.stats.schedule_seconds += t1 - t0
        if ahead:
            rows_before = self._inflight[2] if self._inflight is not None else {}
            entries, prev_rows = [], []
            for item in scheduled:
                r = item.request
                row = rows_before.get(r.id, -1) if item.q_start >= len(r.token_ids) else -1
                if row < 0 and item.q_start >= len(r.token_ids):
                    raise EngineError(f"request {r.id}: the token at position {item.q_start} is not known yet")
                entries.append(StepEntry(r.id, [None] if row >= 0 else [r.token_ids[item.q_start]], item.q_start, [0],
                                         r.params.temperature))
                prev_rows.append(row)
            pending = self.executor.decode_launch(entries, prev_rows)
            self.scheduler.advance(scheduled)
            before, self._inflight = self._inflight, (scheduled, pending, {x.request.id: i for i, x in enumerate(scheduled)})
            self.last_scheduled = scheduled
            self.last_emitted = []
            if before is not None:
                finished = self._resolve(before[0], self.executor.decode_collect(before[1]))
            self.stats.execute_seconds += time.perf_counter() - t1
            return finished
        entries = []
        for item in scheduled:
            r = item.request
            tokens = r.token_ids[item.q_start:item.q_start + item.q_len]
            entries.append(StepEntry(r.id, tokens, item.q_start, [item.q_len - 1] if item.emits() else [],
                                     r.params.temperature))
        out = self.executor.step(entries, sample=True, return_logits=False)
        self.scheduler.advance(scheduled)
        self.last_scheduled = scheduled
        finished += self._resolve(scheduled, out.token_ids)
        self.last_emitted = emitted_before + self.last_emitted
        self.stats.execute_seconds += time.perf_counter() - t1
        return finished

    def _read_inflight(self) -> int:
        """Wait for the step that is still running and take its tokens."""
        scheduled, pending, _ = self._inflight
        self._inflight = None
        return self._resolve(scheduled, self.executor.decode_collect(pending))

    def _resolve(self, scheduled: Sequence[Scheduled], token_ids: Sequence[int]) -> int:
        """Hand a step's tokens to the scheduler; `last_emitted` lists those that count."""
        now = time.perf_counter()
        emitting = [x for x in scheduled if x.emits()]
        lengths = [len(x.request.token_ids) for x in emitting]
        finished = self.scheduler.resolve(scheduled, token_ids)
        self.last_emitted = []
        for x, n_before, token in zip(emitting, lengths, token_ids):
            r = x.request
            if len(r.token_ids) == n_before:
                continue                    # dropped: the request had ended before this step's token
            if r.first_token_time == 0.0:
                r.first_token_time = now
            r.token_times.append(now)
            self.last_emitted.append((r, token))
            if r.status == FINISHED and r.finish_time == 0.0:
                r.finish_time = now
        return finished

    def is_finished(self) -> bool:
        return self.scheduler.is_finished() and self._inflight is None

    def run_until_done(self) -> None:
        while not self.is_finished():
            self.step()

    def release_finished(self) -> None:
        self.requests = [r for r in self.requests if r.status != FINISHED]
        self.last_scheduled = []
        self.last_emitted = []

    def shutdown(self) -> None:
        """Give back what unfinished requests still hold (src/runner/engine.zig:74-84)."""
        if self._inflight is not None:
            self._read_inflight()
        for r in self.requests:
            self.executor.release(r.id)
