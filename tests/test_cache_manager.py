"""The cache manager: no page lost, held twice or freed twice, under random orders (no GPU)."""
import random

import pytest

from llmgen_b200.cache import FULL, WINDOW, CacheError, CacheGroup, CacheManager, GroupSpec, PagePool, StateSlots


def test_pool_hands_out_ascending_ids_and_reuses_lifo():
    p = PagePool(4)
    assert p.take(3) == [0, 1, 2]
    assert p.take(2) is None and p.num_free == 1      # all or nothing
    p.give([2, 1])
    assert p.take(2) == [1, 2]                        # last given back comes first
    with pytest.raises(CacheError, match="freed twice"):
        p.give([3])
    with pytest.raises(CacheError, match="does not belong"):
        p.give([9])


def test_reserve_release_like_the_reference_block_manager():
    # mirrors src/runner/block.zig:82-117: 4 pages of 16 tokens
    m = CacheManager([GroupSpec(FULL)], [4], 16, 8)
    assert m.admit("a") == 0
    assert m.reserve("a", 0, 17) and m.groups[0].table("a") == [0, 1]
    assert m.reserve("a", 17, 32) and m.groups[0].table("a") == [0, 1]      # already covered
    assert m.can_reserve("b", 0, 32) and not m.can_reserve("b", 0, 33)
    assert m.admit("b") == 1
    assert not m.reserve("b", 0, 33) and m.groups[0].table("b") == []       # no side effect
    assert m.reserve("b", 0, 20)
    assert m.groups[0].slot_of("a", 17) == 1 * 16 + 1 and m.groups[0].slot_of("b", 3) == 2 * 16 + 3
    m.release("a")
    assert m.num_free_pages() == [2]
    assert m.reserve("b", 20, 64) and m.groups[0].table("b") == [2, 3, 0, 1]  # freed pages are used again, in their old order
    m.release("b")
    assert m.all_free()


def test_window_group_gives_pages_back_as_the_window_passes():
    g = CacheGroup(GroupSpec(WINDOW, 20), 6, 8)
    assert g.reserve("r", 0, 30)                       # pages 0..3
    assert g.pages_held("r") == 4
    # next token is 30: oldest needed position 11 -> page 0 (positions 0..7) can go
    assert g.reserve("r", 30, 31) and g.table("r")[0] == -1 and g.pages_held("r") == 3
    with pytest.raises(CacheError, match="given back"):
        g.slot_of("r", 3)
    assert g.slot_of("r", 30) == g.table("r")[3] * 8 + 6
    # a long decode never holds more than ceil((W - 1 + 1) / 8) + 1 pages
    for pos in range(31, 400):
        assert g.reserve("r", pos, pos + 1)
        assert g.pages_held("r") <= 4
        first_needed = pos - 20 + 1
        assert all(g.table("r")[i] >= 0 for i in range(first_needed // 8, pos // 8 + 1))
    g.release("r")
    assert g.pool.num_free == 6


def test_window_group_counts_pages_it_can_give_back():
    g = CacheGroup(GroupSpec(WINDOW, 8), 3, 8)
    assert g.reserve("r", 0, 24) and g.pool.num_free == 0
    # positions 24..31 need a 4th page index; page 0 and 1 are out of the window by then
    assert g.can_reserve("r", 24, 32) and g.reserve("r", 24, 32)
    assert g.pages_held("r") == 2


def test_groups_are_all_or_nothing():
    m = CacheManager([GroupSpec(FULL), GroupSpec(WINDOW, 16)], [4, 2], 16, 4)
    m.admit("a")
    assert m.reserve("a", 0, 32)
    assert not m.reserve("a", 32, 80)          # the full group lacks a page; the window group must not change
    assert m.groups[1].table("a") == [0, 1] and m.groups[0].table("a") == [0, 1]
    m.check_consistency()


def test_state_slots():
    s = StateSlots(2)
    assert s.take("a") == 0 and s.take("a") == 0 and s.take("b") == 1 and s.take("c") is None
    s.give("a")
    s.give("a")
    assert s.take("c") == 0 and s.num_free == 0
    m = CacheManager([GroupSpec(FULL)], [2], 16, 1)
    assert m.admit("x") == 0 and m.fresh_state == [0] and m.admit("x") == 0 and m.fresh_state == [0]
    assert m.admit("y") is None
    m.release("x")
    assert m.admit("y") == 0 and m.fresh_state == [0, 0]


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    specs = [GroupSpec(FULL), GroupSpec(WINDOW, rng.choice([8, 24, 50]))]
    m = CacheManager(specs, [rng.randint(8, 20), rng.randint(6, 12)], rng.choice([4, 8, 16]), 5)
    live = {}
    next_id = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            rid = next_id
            next_id += 1
            assert m.admit(rid) is not None
            live[rid] = 0
        elif action < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 7, 33])
            before = [list(g.table(rid)) for g in m.groups]
            free_before = m.num_free_pages()
            could = m.can_reserve(rid, live[rid], live[rid] + n)
            ok = m.reserve(rid, live[rid], live[rid] + n)
            assert ok == could
            if ok:
                live[rid] += n
                for g in m.groups:   # every position the next token attends to has a page
                    lo = g.first_needed_position(live[rid] - 1)
                    assert all(g.table(rid)[i] >= 0 for i in range(lo // m.page_size, (live[rid] - 1) // m.page_size + 1))
            else:
                assert [list(g.table(rid)) for g in m.groups] == before and m.num_free_pages() == free_before
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check_consistency()
    for rid in list(live):
        m.release(rid)
    assert m.all_free()
    with pytest.raises(KeyError):
        m.groups[0].slot_of("nobody", 0)


def test_storage_gives_values_their_own_width_where_a_mixer_asks_for_one():
    """A mixer's `KVRequest` may name another width for values than for keys: the arrays, and the bytes a page
    costs (which the engine's page budget divides by), follow it."""
    import torch
    from llmgen_b200.cache.storage import CacheStorage, bytes_per_page, plan_groups
    from llmgen_b200.parts.base import KVRequest
    reqs = {0: KVRequest(FULL, 0, 2, 48), 1: KVRequest(FULL, 0, 3, 64, v_head_dim=16)}
    groups, index = plan_groups(reqs)
    assert len(groups) == 1 and index == {0: 0, 1: 0}
    page = 8
    assert bytes_per_page(reqs, index, 0, page, torch.bfloat16) == (2 * page * (48 + 48) + 3 * page * (64 + 16)) * 2
    st = CacheStorage(reqs, {}, index, [5], page, 2, torch.float32, "cpu")
    assert st.kv[0][0].shape == (5, 2, page, 48) and st.kv[0][1].shape == (5, 2, page, 48)
    assert st.kv[1][0].shape == (5, 3, page, 64) and st.kv[1][1].shape == (5, 3, page, 16)
    assert st.bytes_held() == 5 * bytes_per_page(reqs, index, 0, page, torch.float32)
    lc = st.layer_cache(1, writes=True)
    assert lc.k.shape[-1] == 64 and lc.v.shape[-1] == 16 and lc.page_size == page
