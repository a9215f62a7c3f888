"""Page allocator and cache manager: no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; state slots."""
import random

import pytest

from velox_b200.cache import CacheGroup, CacheManager, NULL_PAGE, OutOfPagesError, PageAllocator


def test_allocator_order_is_deterministic_and_last_in_first_out():
    alloc = PageAllocator(6)
    assert alloc.num_free == 5 and alloc.num_usable == 5
    assert alloc.take(3) == [1, 2, 3]
    alloc.give_back(2)
    assert alloc.take(2) == [2, 4]
    alloc.give_back(1)
    alloc.give_back(4)
    assert alloc.take(1) == [4]
    alloc.assert_consistent()


def test_allocator_refuses_double_free_and_exhaustion():
    alloc = PageAllocator(4)
    pages = alloc.take(3)
    with pytest.raises(OutOfPagesError):
        alloc.take(1)
    assert alloc.num_free == 0  # a refused request takes nothing
    alloc.give_back(pages[0])
    with pytest.raises(RuntimeError, match="twice"):
        alloc.give_back(pages[0])
    with pytest.raises(IndexError):
        alloc.give_back(9)
    assert alloc.give_back(NULL_PAGE) == 1  # the reserved page is never freed
    assert alloc.share(pages[1]) == 2
    assert alloc.give_back(pages[1]) == 1 and alloc.num_free == 1
    with pytest.raises(RuntimeError):
        alloc.share(pages[0])
    with pytest.raises(ValueError):
        PageAllocator(1)
    alloc.assert_consistent()


def test_tables_grow_by_pages_and_slots_address_tokens():
    manager = CacheManager([CacheGroup("all")], num_pages=10, page_size=4, max_model_len=30, max_num_seqs=2)
    seq = manager.new_sequence("a")
    assert manager.pages_to_append(seq, 5) == 2 and manager.can_append(seq, 5)
    assert manager.append_slots(seq, 5)
    assert seq.tables == [[1, 2]]
    manager.advance(seq, 5)
    assert manager.pages_to_append(seq, 3) == 0 and manager.append_slots(seq, 3)
    assert manager.pages_to_append(seq, 4) == 1
    assert manager.slot_for(seq, 0, 0) == 4 and manager.slot_for(seq, 0, 6) == 2 * 4 + 2
    assert not manager.append_slots(seq, 26)  # beyond max_model_len
    assert seq.tables == [[1, 2]]
    manager.free(seq)
    assert manager.num_free_pages() == 9 and seq.tables == [[]]
    manager.assert_consistent()


def test_max_model_len_is_clamped_to_the_pool():
    manager = CacheManager([CacheGroup("all")], num_pages=24, page_size=8, max_model_len=4096)
    assert manager.max_model_len == 184 and manager.max_blocks_per_seq == 23


def test_append_is_all_groups_or_none():
    manager = CacheManager([CacheGroup("all"), CacheGroup("w", window=8)], num_pages=5, page_size=4, max_model_len=64)
    a = manager.new_sequence("a")
    assert manager.append_slots(a, 12)  # 3 of 4 pages in both pools
    b = manager.new_sequence("b")
    assert not manager.append_slots(b, 8)
    assert b.tables == [[], []]
    assert [alloc.num_free for alloc in manager.allocators] == [1, 1]


def test_window_group_gives_pages_back_as_the_window_passes():
    manager = CacheManager([CacheGroup("all"), CacheGroup("w", window=6)], num_pages=20, page_size=4, max_model_len=64)
    seq = manager.new_sequence("a")
    assert manager.append_slots(seq, 10)
    manager.advance(seq, 10)
    # next query at 10 sees keys 5..10: block 0 (0..3) is dead, block 1 (4..7) is not
    assert seq.tables[1][0] == NULL_PAGE and seq.tables[1][1] != NULL_PAGE
    assert seq.first_live == [0, 1]
    assert all(page != NULL_PAGE for page in seq.tables[0])
    assert manager.allocators[0].num_used == 3 and manager.allocators[1].num_used == 2
    for _ in range(10):
        assert manager.append_slots(seq, 1)
        manager.advance(seq, 1)
        manager.assert_consistent()
    # 20 computed: keys 15..20 are needed -> blocks 0..2 dead
    assert seq.first_live[1] == 3 and manager.allocators[1].num_used == len(seq.tables[1]) - 3
    manager.free(seq)
    assert [alloc.num_used for alloc in manager.allocators] == [0, 0]
    manager.assert_consistent()


def test_state_slots_are_first_in_first_out_with_callbacks():
    manager = CacheManager([CacheGroup("all")], num_pages=8, page_size=4, max_num_seqs=2)
    events = []
    manager.on_slot_acquired = lambda seq: events.append(("got", seq.seq_id, seq.slot))
    manager.on_slot_released = lambda seq: events.append(("gave", seq.seq_id, seq.slot))
    a, b, c = (manager.new_sequence(n) for n in "abc")
    assert manager.acquire_slot(a) and manager.acquire_slot(b)
    assert (a.slot, b.slot) == (0, 1)
    assert manager.acquire_slot(a) and a.slot == 0  # idempotent
    assert not manager.acquire_slot(c)
    manager.release_slot(a)
    assert a.slot is None and manager.acquire_slot(c) and c.slot == 0
    manager.release_slot(a)  # nothing to give back
    assert events == [("got", "a", 0), ("got", "b", 1), ("gave", "a", 0), ("got", "c", 0)]


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window", [None, 10])
def test_random_orders_never_lose_or_double_hold_a_page(seed, window):
    rng = random.Random(seed)
    groups = [CacheGroup("all")] + ([CacheGroup("w", window=window)] if window else [])
    manager = CacheManager(groups, num_pages=33, page_size=4, max_model_len=80, max_num_seqs=6)
    live = {}
    counter = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 6:
            seq = manager.new_sequence(f"s{counter}")
            counter += 1
            assert manager.acquire_slot(seq)
            live[seq.seq_id] = seq
        elif action < 0.8 and live:
            seq = rng.choice(list(live.values()))
            n = rng.choice([1, 1, 1, 2, 5, 9, 17])
            free_before = [alloc.num_free for alloc in manager.allocators]
            if manager.can_append(seq, n):
                assert manager.append_slots(seq, n)
                manager.advance(seq, n)
            else:
                assert not manager.append_slots(seq, n) or seq.num_computed + n <= manager.max_model_len
                if not manager.can_append(seq, n):
                    assert [alloc.num_free for alloc in manager.allocators] == free_before
        elif action < 0.9 and live:
            seq = live.pop(rng.choice(list(live)))
            manager.free(seq)
            manager.release_slot(seq)
        elif live:
            seq = rng.choice(list(live.values()))
            manager.reset_for_recompute(seq)
            assert seq.num_computed == 0
        manager.assert_consistent()
    for seq in live.values():
        manager.free(seq)
        manager.release_slot(seq)
    manager.assert_consistent()
    assert all(alloc.num_used == 0 for alloc in manager.allocators)
    assert manager.num_free_slots == 6


def test_consistency_check_catches_a_lost_page():
    manager = CacheManager([CacheGroup("all")], num_pages=8, page_size=4)
    seq = manager.new_sequence("a")
    manager.append_slots(seq, 9)
    seq.tables[0].pop()  # the table forgets a page the allocator still counts as held
    with pytest.raises(AssertionError, match="lost"):
        manager.assert_consistent()
