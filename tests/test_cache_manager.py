"""The cache manager: pages, tables, reference counts, prefix hash, copy-on-write,
windows, groups and state slots.  Unit rules follow the reference's tests
(tests/test_block_manager.py) with the additions of this engine; the random
test checks that no page is ever lost, held twice or freed twice."""

import random

import pytest

from paged_llm_b200.cache import CacheManager, GroupSpec
from paged_llm_b200.config import SamplingParams
from paged_llm_b200.engine.sequence import NO_PAGE, Sequence


def seq(tokens):
    return Sequence(list(tokens), SamplingParams())


def computed(cm, s, n):
    before = s.num_computed_tokens
    s.num_computed_tokens += n
    cm.cache_full_blocks(s, before, s.num_computed_tokens)
    cm.release_behind_window(s)


def test_allocate_free_round_trip_and_slots():
    cm = CacheManager(8, 4)
    s = seq(range(10))
    new = cm.allocate_slots(s, 10)
    assert new == s.block_table and len(new) == 3 and cm.num_free_blocks == 5
    assert cm.slot_mapping(s, 3, 3) == [new[0] * 4 + 3, new[1] * 4, new[1] * 4 + 1]
    cm.free(s)
    assert cm.num_free_blocks == 8 and s.block_table == []
    cm.check_invariants([])


def test_exhaustion_changes_nothing():
    cm = CacheManager(2, 4)
    s = seq(range(9))
    assert cm.allocate_slots(s, 9) is None
    assert s.block_table == [] and cm.num_free_blocks == 2
    assert cm.allocate_slots(s, 8) is not None


def test_decode_appends_into_the_partial_page():
    cm = CacheManager(8, 4, enable_prefix_caching=False)
    s = seq(range(5))
    cm.allocate_slots(s, 5)
    computed(cm, s, 5)
    for _ in range(3):
        s.append_token(1)
        assert cm.allocate_slots(s, 1) == []
        computed(cm, s, 1)
    s.append_token(1)
    assert len(cm.allocate_slots(s, 1)) == 1


def test_prefix_hit_shares_pages_and_never_covers_the_last_token():
    cm = CacheManager(16, 4)
    a = seq(range(12))
    cm.allocate_slots(a, 12)
    computed(cm, a, 12)
    b = seq(list(range(12)))
    hits, n = cm.get_computed_blocks(b)
    assert n == 8 and hits == a.block_table[:2]            # 12 tokens: only 2 full pages may hit
    assert cm.allocate_slots(b, 4, hits) is not None
    assert b.block_table[:2] == a.block_table[:2] and cm.blocks[hits[0]].ref_count == 2
    cm.check_invariants([a, b])
    cm.free(a)
    cm.free(b)
    # still cached while free, and counted against capacity when hit again
    c = seq(list(range(12)) + [99])
    hits, n = cm.get_computed_blocks(c)
    assert n == 12
    free_before = cm.num_free_blocks
    assert cm.allocate_slots(c, 1, hits) is not None
    assert cm.num_free_blocks == free_before - 4
    assert cm.num_cache_hits == 2 and cm.num_cache_queries == 2


def test_hit_is_confirmed_by_tokens_and_chain_depends_on_the_prefix():
    cm = CacheManager(16, 4)
    a = seq([1, 2, 3, 4, 5, 6, 7, 8, 9])
    cm.allocate_slots(a, 9)
    computed(cm, a, 9)
    b = seq([9, 9, 9, 9, 5, 6, 7, 8, 9])                   # same second page, other first page
    assert cm.get_computed_blocks(b) == ([], 0)


def test_free_cached_pages_count_against_capacity():
    cm = CacheManager(4, 4)
    a = seq(range(8))
    cm.allocate_slots(a, 8)
    computed(cm, a, 8)
    cm.free(a)
    b = seq(list(range(8)) + [1, 2, 3, 4, 5, 6, 7, 8, 9])   # hits 2 pages, needs 3 more: only 2 are free
    hits, n = cm.get_computed_blocks(b)
    assert n == 8
    assert cm.allocate_slots(b, 9, hits) is None
    assert cm.num_free_blocks == 4 and b.block_table == []


def test_lru_eviction_order():
    cm = CacheManager(4, 4)
    a, b = seq(range(8)), seq(range(100, 108))
    cm.allocate_slots(a, 8); computed(cm, a, 8)
    cm.allocate_slots(b, 8); computed(cm, b, 8)
    a_pages = list(a.block_table)
    cm.free(a)
    cm.free(b)
    c = seq(range(200, 204))
    got = cm.allocate_slots(c, 4)
    assert got == [a_pages[1]]                              # freed first, deepest page first
    assert cm.num_cached_blocks == 3


def test_fork_and_copy_on_write():
    cm = CacheManager(8, 4, enable_prefix_caching=False)
    parent = seq(range(6))
    cm.allocate_slots(parent, 6)
    computed(cm, parent, 6)
    child = seq(range(6))
    cm.fork(parent, child)
    assert child.block_table == parent.block_table and cm.blocks[parent.block_table[1]].ref_count == 2
    child.append_token(7)
    shared = child.block_table[1]
    new = cm.allocate_slots(child, 1)
    copies = cm.take_pending_copies()
    assert len(copies) == 1 and copies[0].src == shared and copies[0].dst == child.block_table[1] == new[-1]
    assert cm.blocks[shared].ref_count == 1 and cm.take_pending_copies() == []
    cm.check_invariants([parent, child])
    # no copy when the write starts on a page edge
    p2 = seq(range(8)); cm.allocate_slots(p2, 8); computed(cm, p2, 8)
    c2 = seq(range(8)); cm.fork(p2, c2); c2.append_token(1)
    cm.allocate_slots(c2, 1)
    assert cm.take_pending_copies() == []


def test_copy_on_write_without_a_free_page_rolls_back():
    cm = CacheManager(2, 4, enable_prefix_caching=False)
    parent = seq(range(6)); cm.allocate_slots(parent, 6); computed(cm, parent, 6)
    child = seq(range(6)); cm.fork(parent, child); child.append_token(1)
    assert cm.allocate_slots(child, 1) is None
    assert child.block_table == parent.block_table and cm.take_pending_copies() == []
    cm.check_invariants([parent, child])


def test_double_free_asserts():
    cm = CacheManager(4, 4)
    s = seq(range(4)); cm.allocate_slots(s, 4)
    page = s.block_table[0]
    cm.free(s)
    with pytest.raises(AssertionError, match="double free"):
        cm.pools[0].release(page)


def test_window_group_gives_pages_back_as_the_window_passes():
    cm = CacheManager([GroupSpec(16), GroupSpec(6, window=8)], 4)
    assert not cm.enable_prefix_caching                     # a window drops keys a shared prefix would need
    s = seq(range(40))
    pos = 0
    for n in (10, 3, 1, 1, 7, 2):
        assert cm.allocate_slots(s, n) is not None
        computed(cm, s, n)
        pos += n
        full, win = s.block_tables
        assert NO_PAGE not in full and len(full) == -(-pos // 4)
        first_needed = pos - 8 + 1
        for j, page in enumerate(win):
            assert (page == NO_PAGE) == ((j + 1) * 4 <= first_needed), (pos, j, win)
        cm.check_invariants([s])
    assert cm.num_free_in_group(1) >= 6 - 3                 # never more than ceil(8/4)+1 pages held
    cm.free(s)
    assert cm.num_free_in_group(0) == 16 and cm.num_free_in_group(1) == 6


def test_all_or_nothing_across_groups():
    cm = CacheManager([GroupSpec(8), GroupSpec(1)], 4)
    s = seq(range(8))
    assert cm.allocate_slots(s, 8) is None
    assert s.block_tables == [[], []] and cm.num_free_in_group(0) == 8


def test_state_slots():
    cm = CacheManager(4, 4, num_state_slots=2)
    assert not cm.enable_prefix_caching
    a, b, c = seq([1]), seq([2]), seq([3])
    assert cm.acquire_state_slot(a) and cm.acquire_state_slot(b)
    assert {a.state_slot, b.state_slot} == {0, 1}
    assert not cm.acquire_state_slot(c)
    cm.free(a)
    assert a.state_slot is None and cm.acquire_state_slot(c) and cm.num_free_state_slots == 0


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_books(seed):
    """Admit, grow, fork, preempt and finish requests in random order, with
    shared prefixes, with and without a windowed group: after every operation
    every page is free or held exactly as often as its count says."""
    rng = random.Random(seed)
    bs = rng.choice([2, 4, 8])
    windowed = seed % 2 == 1
    groups = [GroupSpec(24)] + ([GroupSpec(10, window=rng.choice([3, 8, 13]))] if windowed else [])
    cm = CacheManager(groups, bs, enable_prefix_caching=not windowed)
    prefixes = [[rng.randrange(50) for _ in range(rng.randrange(1, 30))] for _ in range(3)]
    live: list[Sequence] = []
    for _ in range(600):
        op = rng.random()
        if op < 0.3 or not live:
            toks = list(rng.choice(prefixes)) + [rng.randrange(50) for _ in range(rng.randrange(1, 12))]
            s = seq(toks)
            hits, n = cm.get_computed_blocks(s)
            want = rng.randrange(1, s.num_tokens - n + 1)
            if cm.allocate_slots(s, want, hits) is not None:
                s.num_computed_tokens = n
                computed(cm, s, want)
                live.append(s)
        elif op < 0.75:
            s = rng.choice(live)
            if s.num_uncomputed_tokens == 0:
                s.append_token(rng.randrange(50))
            n = rng.randrange(1, s.num_uncomputed_tokens + 1)
            if cm.allocate_slots(s, n) is not None:
                computed(cm, s, n)
            cm.take_pending_copies()
        elif op < 0.85 and not windowed:
            parent = rng.choice(live)
            child = seq(parent.token_ids)
            cm.fork(parent, child)
            live.append(child)
        elif op < 0.92:
            s = rng.choice(live)                            # preempt: pages back, request stays
            cm.free(s)
            s.reset_for_recompute()
            live.remove(s)
        else:
            s = rng.choice(live)
            cm.free(s)
            live.remove(s)
        cm.check_invariants(live)
    for s in live:
        cm.free(s)
    cm.check_invariants([])
    assert all(len(p.free) == p.num_pages for p in cm.pools)
