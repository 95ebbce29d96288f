"""The C++ host runtime against its plain restatement: the same random operations on both, and
every observable (tables, free lists, state slots, schedules, request fields) must agree."""
import ctypes
import random

import numpy as np
import pytest

from llmgen_b200.cache import FULL, WINDOW, CacheManager, GroupSpec
from llmgen_b200.cache.manager import runtime
from llmgen_b200.engine.scheduler import CHUNKED, FINISHED, PREFILL_FIRST, BatchScheduler, Request, SchedulerConfig
from llmgen_b200.sampling import SamplingParams
from tests.plain import runtime_plain as plain


def both(specs, pages, page_size, slots):
    native = CacheManager([GroupSpec(k, w) for k, w in specs], pages, page_size, slots)
    oracle = plain.CacheManager([plain.GroupSpec(k, w) for k, w in specs], pages, page_size, slots)
    return native, oracle


def same_state(native, oracle, reqs):
    assert native.num_free_pages() == oracle.num_free_pages()
    assert native.state.num_free == oracle.state.num_free
    for gn, go in zip(native.groups, oracle.groups):
        assert gn.pool.free_list() == go.pool._free
        assert gn.num_tables == len(go.tables)
        for r in reqs:
            assert gn.table(r) == go.tables.get(r, [])
    for r in reqs:
        assert native.is_admitted(r) == oracle.is_admitted(r)
        if oracle.is_admitted(r):
            assert native.state.slot(r) == oracle.state.owner[r]
    assert list(native.fresh_state) == list(oracle.fresh_state)


@pytest.mark.parametrize("seed", range(6))
def test_cache_manager_follows_the_plain_one(seed):
    rng = random.Random(seed)
    page_size = rng.choice([4, 8, 16])
    window = rng.choice([5, 9, 24])
    specs = [(FULL, 0), (WINDOW, window)] if seed % 2 else [(FULL, 0)]
    pages = [rng.randint(6, 14) for _ in specs]
    native, oracle = both(specs, pages, page_size, 3)
    reqs = ["a", 1, ("b", 2), 7]                      # names of several kinds, ints among them
    length = {r: 0 for r in reqs}
    for _ in range(400):
        r = rng.choice(reqs)
        op = rng.random()
        if op < 0.2:
            assert native.admit(r) == oracle.admit(r)
        elif op < 0.7:
            if not oracle.is_admitted(r):
                continue
            n = rng.randint(1, 2 * page_size)
            start, end = length[r], length[r] + n
            assert native.can_reserve(r, start, end) == oracle.can_reserve(r, start, end)
            ok = oracle.reserve(r, start, end)
            assert native.reserve(r, start, end) == ok
            if ok:
                length[r] = end
        elif op < 0.8:
            native.release_pages(r)
            oracle.release_pages(r)
            length[r] = 0
        elif op < 0.95:
            native.release(r)
            oracle.release(r)
            length[r] = 0
        else:
            native.fresh_state.clear()
            oracle.fresh_state.clear()
        same_state(native, oracle, reqs)
        native.check_consistency()
    for r in reqs:
        native.release(r)
        oracle.release(r)
    assert native.all_free() and oracle.all_free()


def drive(make_scheduler, make_cache, seed, policy):
    rng = random.Random(seed)
    cache = make_cache(rng.randint(10, 18))
    s = make_scheduler(cache, SchedulerConfig(policy=policy, chunk_tokens=rng.choice([8, 16, 64]),
                                              max_num_batched_tokens=rng.choice([72, 96]), max_num_seqs=4,
                                              eos_token_ids=(3,)))
    reqs = [Request(i, list(range(1, rng.randint(1, 30) + 1)),
                    SamplingParams(temperature=0.0, max_tokens=rng.randint(1, 40), ignore_eos=rng.random() < 0.5))
            for i in range(14)]
    pending = list(reqs)
    log = []
    steps = 0
    while pending or not s.is_finished():
        if pending and rng.random() < 0.3:
            s.add(pending.pop(0))
        if s.is_finished():
            continue
        sched = s.schedule()
        steps += 1
        assert steps < 5000
        tokens = [rng.randrange(20) for x in sched if x.emits()]
        log.append(([(x.request.id, x.q_start, x.q_len) for x in sched],
                    [r.id for r in s.waiting], [r.id for r in s.running], s.num_preemptions))
        s.postprocess(sched, tokens)
        log.append([(r.status, r.num_computed_tokens, r.num_preemptions, len(r)) for r in reqs])
        log.append(cache.num_free_pages())
    assert all(r.status == FINISHED for r in reqs) and cache.all_free()
    return log, [r.token_ids for r in reqs]


@pytest.mark.parametrize("policy", [PREFILL_FIRST, CHUNKED])
@pytest.mark.parametrize("seed", range(5))
def test_scheduler_follows_the_plain_one(policy, seed):
    native = drive(BatchScheduler, lambda n: CacheManager([GroupSpec(FULL)], [n], 8, 4), seed, policy)
    oracle = drive(plain.PlainBatchScheduler, lambda n: plain.CacheManager([plain.GroupSpec(FULL)], [n], 8, 4),
                   seed, policy)
    assert native[0] == oracle[0]
    assert native[1] == oracle[1]


def test_scheduler_takes_an_executor_like_owner_of_the_cache_and_refuses_anything_else():
    class Owner:
        def __init__(self, cache):
            self.cache = cache

    cache = CacheManager([GroupSpec(FULL)], [8], 8, 2)
    s = BatchScheduler(Owner(cache), SchedulerConfig())
    r = Request(0, [1, 2, 3], SamplingParams(temperature=0.0, max_tokens=1))
    s.add(r)
    sched = s.schedule()
    assert [(x.q_start, x.q_len) for x in sched] == [(0, 3)] and list(cache.fresh_state) == [0]
    assert s.postprocess(sched, [9]) == 1 and cache.all_free()
    with pytest.raises(Exception, match="CacheManager"):
        BatchScheduler(object(), SchedulerConfig())
    with pytest.raises(Exception, match="generated"):
        s.add(r)                                   # it has a completion: only fresh requests are added
    again = Request(1, [1, 2], SamplingParams(temperature=0.0, max_tokens=1))
    s.add(again)
    with pytest.raises(Exception, match="already"):
        s.add(again)


def test_decode_step_arrays_are_filled_natively_and_rows_rewritten_only_when_a_table_changed():
    """`llmr_fill_decode` writes ids, positions, lengths, state slots, temperatures, cache slots and
    block-table rows of a step of single tokens; compared here with the tables themselves."""
    lib = runtime()
    page_size, max_blocks, bucket = 4, 6, 4
    cache = CacheManager([GroupSpec(FULL), GroupSpec(WINDOW, 6)], [16, 16], page_size, 4)
    lengths = {10: 9, 11: 4, 12: 17}
    for r, n in lengths.items():
        assert cache.admit(r) is not None and cache.reserve(r, 0, n + 1)
    words = 8 * bucket + 2 * (bucket + bucket * max_blocks)
    host = (ctypes.c_int * words)()
    offs, at = [], 0
    for size in [bucket] * 6 + [2 * bucket] + [bucket, bucket * max_blocks] * 2:
        offs.append(at)
        at += size
    offs_c = (ctypes.c_int * len(offs))(*offs)
    stamps = (ctypes.c_longlong * (2 * 2 * bucket))()

    def fill(reqs, tokens, starts, temps, rows_before=None):
        n = len(reqs)
        rc = lib.llmr_fill_decode(cache.native_handle, host, offs_c, ctypes.c_int(n), ctypes.c_int(bucket),
                                  ctypes.c_int(max_blocks), (ctypes.c_longlong * n)(*[cache.key(r) for r in reqs]),
                                  (ctypes.c_int * n)(*tokens), (ctypes.c_int * n)(*(rows_before or [-1] * n)),
                                  (ctypes.c_int * n)(*starts), (ctypes.c_float * n)(*temps), ctypes.c_ulonglong(SEED), stamps)
        return rc, np.frombuffer(host, dtype=np.int32).copy()

    SEED, STRIDE, M64 = 0x5EED5EED5EED, 0x9E3779B97F4A7C15, (1 << 64) - 1
    reqs = [10, 11, 12]
    starts = [lengths[r] for r in reqs]
    rc, a = fill(reqs, [5, 6, 7], starts, [0.0, 0.5, 1.0])
    assert rc == 0
    # the sampler's key of a row: the request and the position, not the row or the number of steps
    keys = a[offs[6]:offs[6] + 8].view(np.uint64).tolist()
    assert keys == [((SEED + STRIDE * (p + 1)) & M64) ^ ((r << 40) & M64) for r, p in zip(reqs, starts)] + [0]
    assert a[offs[0]:offs[0] + 4].tolist() == [5, 6, 7, 0]
    assert a[offs[1]:offs[1] + 4].tolist() == starts + [0]
    assert a[offs[2]:offs[2] + 4].tolist() == [s + 1 for s in starts] + [0]
    assert a[offs[3]:offs[3] + 4].tolist() == [cache.state.slot(r) for r in reqs] + [-1]
    assert a[offs[4]:offs[4] + 4].view(np.float32).tolist() == [0.0, 0.5, 1.0, 0.0]
    assert a[offs[5]:offs[5] + 4].tolist() == [-1, -1, -1, -1]
    for g, group in enumerate(cache.groups):
        slots = a[offs[7 + 2 * g]:offs[7 + 2 * g] + 4].tolist()
        assert slots == [group.slot_of(r, p) for r, p in zip(reqs, starts)] + [-1]
        rows = a[offs[8 + 2 * g]:offs[8 + 2 * g] + bucket * max_blocks].reshape(bucket, max_blocks)
        for s, r in enumerate(reqs):
            t = group.table(r)
            assert rows[s, :len(t)].tolist() == t and not rows[s, len(t):].any()
        assert not rows[3].any()
    # a row that holds the same table at the same length is left alone (its stamp matches) ...
    host[offs[8] + 0] = 999
    rc, a = fill(reqs, [5, 6, 7], starts, [0.0, 0.5, 1.0])
    assert rc == 0 and a[offs[8] + 0] == 999
    # ... and written again once the table has grown, or when another request takes the row
    assert cache.reserve(10, lengths[10] + 1, lengths[10] + 1 + page_size)
    rc, a = fill(reqs, [5, 6, 7], starts, [0.0, 0.5, 1.0])
    assert rc == 0 and a[offs[8]:offs[8] + max_blocks].tolist()[:len(cache.groups[0].table(10))] == cache.groups[0].table(10)
    rc, a = fill([12, 11], [1, 2], [lengths[12], lengths[11]], [0.0, 0.0])
    t = cache.groups[0].table(12)
    assert rc == 0 and a[offs[8]:offs[8] + len(t)].tolist() == t
    assert not a[offs[8] + 2 * max_blocks:offs[8] + 3 * max_blocks].any()        # row 2 is padding now
    # ids that are still on the device: the row of the step before is passed on, the id left at zero
    rc, a = fill(reqs, [5, 6, 7], starts, [0.0, 0.5, 1.0], rows_before=[2, -1, 0])
    assert rc == 0 and a[offs[0]:offs[0] + 4].tolist() == [0, 6, 0, 0] and a[offs[5]:offs[5] + 4].tolist() == [2, -1, 0, -1]
    # a position without a page is refused with a message
    rc, _ = fill([11], [1], [lengths[11] + 2 * page_size], [0.0])
    assert rc == 1 and b"no page" in lib.llmr_last_error()
