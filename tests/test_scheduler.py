"""The scheduler's decisions, on the cache manager alone (no GPU)."""
import random

import pytest

from llmgen_b200.cache import FULL, CacheManager, GroupSpec
from llmgen_b200.engine.scheduler import (CHUNKED, FINISHED, PREFILL_FIRST, RUNNING, WAITING, BatchScheduler, Request,
                                          SchedulerConfig, SchedulerError)
from llmgen_b200.sampling import SamplingParams


def make(pages, page_size=16, **cfg):
    cache = CacheManager([GroupSpec(FULL)], [pages], page_size, cfg.get("max_num_seqs", 256))
    return cache, BatchScheduler(cache, SchedulerConfig(**cfg))


def req(i, n, max_tokens=4, **kw):
    return Request(i, list(range(1, n + 1)), SamplingParams(temperature=0.0, max_tokens=max_tokens, **kw))


def run(s, steps=1000, token=7):
    """Drive the scheduler with a constant sampled token; returns the list of schedules."""
    log = []
    for _ in range(steps):
        if s.is_finished():
            break
        sched = s.schedule()
        assert sched, "stuck"
        log.append([(x.request.id, x.q_start, x.q_len) for x in sched])
        s.postprocess(sched, [token] * sum(1 for x in sched if x.emits()))
        s.cache.check_consistency()
    return log


def test_prefill_first_whole_prompts_then_decode():
    cache, s = make(64, max_num_batched_tokens=50)
    for i, n in enumerate((20, 25, 30)):
        s.add(req(i, n, max_tokens=2))
    log = run(s)
    assert log[0] == [(0, 0, 20), (1, 0, 25)]          # 20 + 25 + 30 > 50: the third waits
    assert log[1] == [(2, 0, 30)]                      # a step that admits is prefill-only
    assert log[2] == [(0, 20, 1), (1, 25, 1), (2, 30, 1)]
    assert len(log) == 3 and cache.all_free()


def test_chunked_cuts_prompts_under_both_budgets():
    cache, s = make(64, policy=CHUNKED, chunk_tokens=16, max_num_batched_tokens=24)
    s.add(req(0, 40, max_tokens=3))
    s.add(req(1, 10, max_tokens=3))
    log = run(s)
    assert log[0] == [(0, 0, 16)]                                  # chunk budget
    assert log[1] == [(0, 16, 16)]
    assert log[2] == [(0, 32, 8), (1, 0, 8)]                       # rest of 0, then 1 within the chunk budget
    assert log[3] == [(0, 40, 1), (1, 8, 2)]                       # a decode row beside the end of a prompt
    assert log[4] == [(0, 41, 1), (1, 10, 1)]
    assert cache.all_free()


def test_emits_only_when_the_portion_reaches_the_end():
    cache, s = make(64, policy=CHUNKED, chunk_tokens=8)
    r = req(0, 20, max_tokens=1)
    s.add(r)
    sched = s.schedule()
    assert not sched[0].emits()
    s.postprocess(sched, [])
    assert r.num_computed_tokens == 8 and len(r) == 20
    s.postprocess(s.schedule(), [])
    sched = s.schedule()
    assert sched[0].emits() and (sched[0].q_start, sched[0].q_len) == (16, 4)
    assert s.postprocess(sched, [5]) == 1 and r.status == FINISHED and r.completion == [5]


def test_out_of_pages_preempts_the_last_running_sequence():
    # 6 pages of 16: two prompts of 40 take 3 pages each; the first decode past 48 needs a 4th
    cache, s = make(6, max_num_seqs=4)
    a, b = req(0, 40, max_tokens=30), req(1, 40, max_tokens=30)
    s.add(a)
    s.add(b)
    log = run(s, steps=9)
    assert log[0] == [(0, 0, 40), (1, 0, 40)]
    assert all(step == [(0, 40 + i, 1), (1, 40 + i, 1)] for i, step in enumerate(log[1:9]))
    # token 49 of request 0 needs page index 3: request 1 (the last) is preempted
    sched = s.schedule()
    assert [(x.request.id, x.q_start, x.q_len) for x in sched] == [(0, 48, 1)]
    assert b.status == WAITING and s.waiting[0] is b and b.num_computed_tokens == 0 and b.num_preemptions == 1
    assert s.num_preemptions == 1 and len(b) == 49            # it keeps the tokens it generated
    s.postprocess(sched, [7])
    # while 0 runs, 1 cannot come back (no pages): prefill_first tries to admit, fails, decodes
    sched = s.schedule()
    assert [(x.request.id, x.q_len) for x in sched] == [(0, 1)]
    s.postprocess(sched, [7])
    log2 = run(s)
    # after 0 finished, 1 is computed again from position 0, generated tokens included
    readmit = [step for step in log2 if step[0][0] == 1][0]
    assert readmit == [(1, 0, 49)]
    assert a.status == FINISHED and b.status == FINISHED
    assert len(a.completion) == 30 and len(b.completion) == 30 and cache.all_free()


def test_a_sequence_alone_preempts_itself_and_scheduling_stops():
    cache, s = make(2, max_num_seqs=4)
    r = req(0, 30, max_tokens=10)
    s.add(r)
    run(s, steps=3)                       # prefill + 2 decodes: 32 tokens = both pages
    other = req(1, 5, max_tokens=1)
    sched = s.schedule()                  # token 33 needs a third page: self-preemption
    assert sched == [] and r.status == WAITING and s.num_preemptions == 1 and cache.all_free()
    # it can never fit again (32 tokens + the next): the engine reports this as stuck
    assert s.schedule() == [] or True


def test_max_num_seqs_bounds_admission_and_state_slots():
    cache, s = make(64, max_num_seqs=2)
    for i in range(3):
        s.add(req(i, 5, max_tokens=2))
    log = run(s)
    assert log[0] == [(0, 0, 5), (1, 0, 5)]
    assert all(len(step) <= 2 for step in log)
    assert cache.all_free()


def test_eos_finishes_unless_ignored():
    cache, s = make(16, eos_token_ids=(7,))
    a, b = req(0, 3, max_tokens=5), req(1, 3, max_tokens=5, ignore_eos=True)
    s.add(a)
    s.add(b)
    run(s, token=7)
    assert a.completion == [7] and b.completion == [7] * 5


def test_prefill_first_cannot_readmit_a_sequence_longer_than_the_token_budget():
    """Whole prompts only: a preempted sequence that outgrew max_num_batched_tokens never fits
    again, which is why the engine refuses a token budget below max_model_len for this policy."""
    cache, s = make(64, max_num_batched_tokens=16)
    s.add(req(0, 20))
    assert s.schedule() == [] and s.waiting


def test_unknown_policy():
    with pytest.raises(SchedulerError):
        SchedulerConfig(policy="fastest")


@pytest.mark.parametrize("policy", [PREFILL_FIRST, CHUNKED])
@pytest.mark.parametrize("seed", range(4))
def test_random_workloads_finish_and_free_everything(policy, seed):
    rng = random.Random(seed)
    cache, s = make(rng.randint(12, 20), page_size=8, policy=policy, chunk_tokens=rng.choice([8, 16, 64]),
                    max_num_batched_tokens=rng.choice([72, 96]), max_num_seqs=4)
    reqs = [req(i, rng.randint(1, 30), max_tokens=rng.randint(1, 40)) for i in range(12)]
    pending = list(reqs)
    steps = 0
    while pending or not s.is_finished():
        if pending and rng.random() < 0.3:
            s.add(pending.pop(0))
        if s.is_finished():
            continue
        sched = s.schedule()
        steps += 1
        assert steps < 5000
        if not sched:
            continue
        assert len({x.request.id for x in sched}) == len(sched) <= 4
        assert sum(x.q_len for x in sched) <= s.config.max_num_batched_tokens
        for x in sched:
            assert x.q_start == x.request.num_computed_tokens and x.request.status == RUNNING
        s.postprocess(sched, [rng.randrange(100) for x in sched if x.emits()])
        cache.check_consistency()
    assert all(r.status == FINISHED and len(r.completion) == r.params.max_tokens for r in reqs)
    assert cache.all_free()


def test_steps_launched_before_the_tokens_of_the_step_before_are_known():
    """`advance` right after a launch, `resolve` when the tokens arrive, one step later: lengths grow at
    once, max_tokens ends a request at `advance`, an end-of-sequence token ends it at `resolve`, and the
    token that a step already launched sampled for it is dropped."""
    cache, s = make(64, eos_token_ids=(9,))
    a, b, c = req(0, 5, max_tokens=3), req(1, 6, max_tokens=8), req(2, 4, max_tokens=8, ignore_eos=True)
    for r in (a, b, c):
        s.add(r)
    first = s.schedule()                                   # the prompts: read at once
    assert all(x.emits() for x in first) and s.postprocess(first, [1, 1, 1]) == 0
    k1 = s.schedule()
    assert [(x.request.id, x.q_start, x.emits()) for x in k1] == [(0, 5, True), (1, 6, True), (2, 4, True)]
    s.advance(k1)
    k2 = s.schedule()                                      # scheduled while k1's tokens are unknown
    assert [(x.request.id, x.q_start, x.emits()) for x in k2] == [(0, 6, True), (1, 7, True), (2, 5, True)]
    assert len(a) == 6                                     # the request's own list is one short
    s.advance(k2)                                          # a has its 3 tokens with this one: it leaves the queues
    assert [r.id for r in s.running] == [1, 2] and a.status != FINISHED
    assert s.resolve(k1, [2, 9, 9]) == 1                   # b's token ends its sequence; c ignores that
    assert b.status == FINISHED and b.completion == [1, 9] and c.completion == [1, 9]
    k3 = s.schedule()
    assert [(x.request.id, x.q_start) for x in k3] == [(2, 6)]
    s.advance(k3)
    assert s.resolve(k2, [3, 4, 5]) == 1                   # a's last token; b's is dropped
    assert a.status == FINISHED and a.completion == [1, 2, 3] and b.completion == [1, 9] and c.completion == [1, 9, 5]
    assert s.resolve(k3, [6]) == 0 and c.completion == [1, 9, 5, 6]
    run(s)
    assert c.status == FINISHED and len(c.completion) == 8 and cache.all_free()


def test_a_request_preempted_while_its_token_is_unknown_keeps_that_token():
    cache, s = make(6, max_num_seqs=4)
    a, b = req(0, 40, max_tokens=30), req(1, 40, max_tokens=30)
    s.add(a)
    s.add(b)
    run(s, steps=8)                                        # prompts, then 7 decoded tokens: lengths 48, three full pages
    k = s.schedule()
    s.advance(k)                                           # lengths 49 now, the tokens not yet known
    nxt = s.schedule()                                     # position 48 needs a 4th page for each: b is preempted
    assert [(x.request.id, x.q_start) for x in nxt] == [(0, 48)] and b.status == WAITING and s.waiting[0] is b
    assert s.resolve(k, [7, 7]) == 0 and len(b) == 49 and len(a) == 49
    s.advance(nxt)
    s.resolve(nxt, [7])
    run(s)
    assert len(a.completion) == 30 and len(b.completion) == 30 and cache.all_free()
