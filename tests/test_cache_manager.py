"""The cache manager's bookkeeping: no page lost, held twice or freed twice, under random orders of requests;
all-or-nothing reservations; windows give pages back; state slots."""

from __future__ import annotations

import random

import pytest
import torch

from liteinfer_b200.cache.manager import CacheManager
from liteinfer_b200.cache.pages import CacheExhaustedError, OutOfPagesError, PageAllocator
from liteinfer_b200.parts.context import KVNeed, StateNeed
from liteinfer_b200.parts.spec import ScheduleEntry


def _manager(needs, schedule=None, page_size=4, num_pages=16, max_requests=4, storage=False):
    schedule = schedule or tuple(ScheduleEntry(i) for i in range(len(needs)))
    return CacheManager(needs, schedule, page_size, num_pages, max_requests, torch.float32, "cpu",
                        allocate_storage=storage)


FULL = (KVNeed(2, 8),)
WINDOW = (KVNeed(2, 8, window=6),)


def test_page_allocator_is_lifo_and_strict():
    pages = PageAllocator(4)
    a = pages.allocate(3)
    assert a == [0, 1, 2] and pages.num_free == 1
    pages.free([1])
    assert pages.allocate(1) == [1]            # the page given back is the next one handed out
    with pytest.raises(OutOfPagesError):
        pages.allocate(2)
    assert pages.num_free == 1                 # a refused allocation takes nothing
    pages.free([0])
    with pytest.raises(ValueError, match="not held"):
        pages.free([0])
    with pytest.raises(ValueError, match="does not exist"):
        pages.free([9])


def test_reserve_is_all_or_nothing_across_requests_and_groups():
    m = _manager([FULL, WINDOW, FULL], num_pages=5)
    assert len(m.groups) == 2 and m.groups[0].stops == [0, 2] and m.groups[1].stops == [1]
    m.reserve(["a"], [9])                      # 3 pages in each group
    m.commit("a", 9)
    with pytest.raises(OutOfPagesError):
        m.reserve(["a", "b"], [10, 12])        # b alone needs 3, only 2 free
    assert not m.has("b") and m.length("a") == 9
    assert [g.allocator.num_free for g in m.groups] == [2, 3]    # the window group already gave one back
    m.check_invariants()
    m.reserve(["a", "b"], [10, 8])
    m.check_invariants()


def test_window_pages_come_back_after_the_window_has_passed():
    m = _manager([WINDOW], page_size=4, num_pages=4)
    total = 0
    for step in range(40):                     # 40 tokens through 4 pages of 4 with a window of 6
        m.reserve(["a"], [total + 1])
        total += 1
        m.commit("a", total)
        table = m.block_table(0, "a")
        first_needed = max(0, total - 6 + 1) // 4
        assert all(p == -1 for p in table[:first_needed]) and all(p >= 0 for p in table[first_needed:])
        assert m.groups[0].allocator.num_held <= 3
        m.check_invariants()
    m.release("a")
    assert m.groups[0].allocator.num_free == 4


def test_a_portion_larger_than_the_window_keeps_what_its_first_query_sees():
    m = _manager([WINDOW], page_size=4, num_pages=8)
    m.reserve(["a"], [10]); m.commit("a", 10)
    held_before = [p for p in m.block_table(0, "a") if p >= 0]
    m.reserve(["a"], [21])                     # the query at position 10 still reads keys 5..10
    assert all(p in m.block_table(0, "a") for p in held_before)
    m.commit("a", 21)
    assert m.block_table(0, "a")[:4] == [-1, -1, -1, -1]


def test_rollback_gives_back_only_the_new_pages():
    m = _manager([FULL], num_pages=8)
    m.reserve(["a"], [6]); m.commit("a", 6)
    m.reserve(["a", "b"], [13, 5])
    m.rollback(["a", "b"])
    assert m.length("a") == 6 and len(m.block_table(0, "a")) == 2 and not m.has("b")
    assert m.groups[0].allocator.num_held == 2 and m.slots.num_held == 1
    m.check_invariants()


def test_state_slots_are_taken_at_admission_zeroed_on_reuse_and_limited():
    needs = [(StateNeed((3,), "f32"),), FULL]
    m = _manager(needs, max_requests=2, storage=True)
    m.reserve(["a", "b"], [1, 1])
    caches = m.layer_caches()
    assert caches[0].state.shape == (2, 3) and caches[0].kv is None and caches[1].kv is not None
    caches[0].state[m.state_slot("a")] = 7.0
    with pytest.raises(CacheExhaustedError, match="state slots"):
        m.reserve(["c"], [1])
    slot = m.state_slot("a")
    m.release("a")
    m.reserve(["c"], [1])
    assert m.state_slot("c") == slot and float(caches[0].state[slot].abs().sum()) == 0.0


def test_schedule_may_share_a_cache_and_repeat_a_layer():
    schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_of=1))
    m = _manager([FULL, FULL], schedule=schedule, storage=True)
    assert m.groups[0].stops == [0, 1, 2] and m.groups[0].pool.shape[0] == 3
    caches = m.layer_caches()
    assert caches[3].read_only and caches[3].kv.k_pool.data_ptr() == caches[1].kv.k_pool.data_ptr()
    assert caches[2].kv.k_pool.data_ptr() != caches[0].kv.k_pool.data_ptr()


def test_misuse_is_refused():
    m = _manager([FULL])
    with pytest.raises(ValueError, match="twice"):
        m.reserve(["a", "a"], [1, 2])
    m.reserve(["a"], [5]); m.commit("a", 5)
    with pytest.raises(ValueError, match="shrink"):
        m.reserve(["a"], [3])
    m.release("zzz")                           # releasing an unknown request is a no-op


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    m = _manager([FULL, WINDOW, (StateNeed((2,)),)], page_size=rng.choice([1, 3, 4, 8]),
                 num_pages=rng.choice([6, 13, 40]), max_requests=4)
    lengths: dict[str, int] = {}
    counter = 0
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and len(lengths) < 6:
            counter += 1
            ids, totals = [f"r{counter}"], [rng.randint(1, 30)]
        elif action < 0.8 and lengths:
            ids = rng.sample(sorted(lengths), rng.randint(1, len(lengths)))
            totals = [lengths[r] + rng.choice([1, 1, 1, 2, 9]) for r in ids]
        elif lengths:
            victim = rng.choice(sorted(lengths))
            m.release(victim)
            del lengths[victim]
            m.check_invariants()
            continue
        else:
            continue
        before = ([g.allocator.num_free for g in m.groups], m.slots.num_free, dict(lengths))
        try:
            m.reserve(ids, totals)
        except CacheExhaustedError:
            assert ([g.allocator.num_free for g in m.groups], m.slots.num_free) == before[:2]
            m.check_invariants()
            continue
        if rng.random() < 0.15:                # the step failed after its reservation
            m.rollback(ids)
            for r in ids:
                assert m.length(r) == before[2].get(r, 0)
        else:
            for r, t in zip(ids, totals):
                m.commit(r, t)
                lengths[r] = t
        m.check_invariants()
        for r, t in lengths.items():
            assert m.length(r) == t
            full = m.block_table(0, r)
            assert len(full) == -(-t // m.page_size) and all(p >= 0 for p in full)
    for r in list(lengths):
        m.release(r)
    assert all(g.allocator.num_held == 0 for g in m.groups) and m.slots.num_held == 0


def test_table_version_moves_exactly_when_a_table_does():
    """A caller may keep a copy of a request's block tables while `table_version` stays the same."""
    cache = _manager([FULL, WINDOW], page_size=4, num_pages=16)

    def snapshot(r):
        return [list(cache.block_table(g, r)) for g in range(len(cache.groups))], cache.state_slot(r)

    cache.reserve(["a"], [3]); cache.commit("a", 3)
    version, seen = cache.table_version("a"), snapshot("a")
    history = {version}
    for total in range(4, 30):
        cache.reserve(["a"], [total])
        cache.commit("a", total)
        if cache.table_version("a") == version:
            assert snapshot("a") == seen
        else:
            assert snapshot("a") != seen and cache.table_version("a") not in history
            version, seen = cache.table_version("a"), snapshot("a")
            history.add(version)
    cache.reserve(["a"], [40])                       # new pages ...
    assert cache.table_version("a") != version
    version = cache.table_version("a")
    cache.rollback(["a"])                            # ... given back: the tables moved again
    assert cache.table_version("a") != version
    cache.release("a")
    cache.reserve(["a"], [2])                        # the same name again is a new request
    assert cache.table_version("a") not in history
    cache.check_invariants()


def test_slot_addressing_follows_the_block_tables():
    """`packed_addresses`, `newest_slots` and `slot_table` name the same places as the block tables the
    kernels read: a token written through a slot is found through (page, position in page)."""
    from liteinfer_b200.cache.addressing import newest_slots, packed_addresses, slot_table

    cache = _manager([FULL], page_size=4, num_pages=16, storage=True)
    cache.reserve(["b"], [5]); cache.commit("b", 5)
    cache.reserve(["a", "b"], [7, 11])
    tables = [cache.block_table(0, r) for r in ("a", "b")]
    packed = packed_addresses(tables, [0, 5], [7, 6], 4)
    assert packed.query_start_loc.tolist() == [0, 7, 13] and packed.context_lens.tolist() == [7, 11]
    assert packed.positions[0].tolist() == [*range(7), *range(5, 11)]
    pool = cache.groups[0].pool[0, 0]                                  # [pages, kv_heads, page_size, head_dim]
    for token, slot in enumerate(packed.slots[0].tolist()):
        pool[slot // 4, :, slot % 4] = token + 1                       # "write" every token of the step
    for i, (start, count) in enumerate(((0, 7), (5, 6))):
        for position in range(start, start + count):
            page = tables[i][position // 4]
            token = int(packed.query_start_loc[i]) + position - start
            assert float(pool[page, 0, position % 4, 0]) == token + 1
    table = slot_table(tables, [7, 11], 4)
    assert table.shape == (2, 11) and table[0, 7:].tolist() == [-1] * 4
    assert table[1, 5:11].tolist() == packed.slots[0, 7:].tolist()
    assert newest_slots(tables, [6, 10], 4).tolist() == [[int(table[0, 6]), int(table[1, 10])]]
    assert len(set(table[table >= 0].tolist())) == 18                  # no slot named twice


def test_a_layer_may_keep_several_named_needs():
    """Two mixers in one block, or a mixer with two states: every need is found under its name; needs that are
    equal apart from the name share a group of pages (and its block tables)."""
    needs = [(KVNeed(2, 8), KVNeed(2, 8, name="cross"), StateNeed((3,), "f32", name="tail"), StateNeed((5, 2), "weight", name="memory")),
             (KVNeed(2, 8),)]
    m = CacheManager(needs, (ScheduleEntry(0), ScheduleEntry(1)), 4, 6, 2, torch.float32, "cpu")
    assert len(m.groups) == 1 and m.groups[0].holders == [(0, "kv"), (0, "cross"), (1, "kv")]
    assert m.groups[0].pool.shape[0] == 3
    first, second = m.layer_caches()
    assert set(first.kvs) == {"kv", "cross"} and set(first.states) == {"tail", "memory"}
    assert first.kvs["kv"].k_pool.data_ptr() != first.kvs["cross"].k_pool.data_ptr()
    assert first.states["tail"].shape == (2, 3) and first.states["memory"].shape == (2, 5, 2)
    assert first.kv is first.kvs["kv"] and first.state is None          # two states, neither named "state"
    assert second.kv is not None and second.state is None and not second.states
    with pytest.raises(ValueError, match="named 'kv'"):
        CacheManager([(KVNeed(2, 8), KVNeed(4, 8))], (ScheduleEntry(0),), 4, 6, 2, torch.float32, "cpu")


def test_a_window_bounds_what_a_request_costs_its_group():
    needs = [(KVNeed(1, 4),), (KVNeed(1, 4, window=10),)]
    m = CacheManager(needs, (ScheduleEntry(0), ScheduleEntry(1)), 4, 12, 8, torch.float32, "cpu", allocate_storage=False)
    full, windowed = m.groups
    assert full.pages_at(40, 8) == 10 and windowed.pages_at(40, 8) == 6 and windowed.pages_at(3, 8) == 1
    assert m.can_hold([40], 8) and not m.can_hold([40, 20], 8)             # the group that keeps all keys decides
    only_window = CacheManager([(KVNeed(1, 4, window=10),)], (ScheduleEntry(0),), 4, 12, 8, torch.float32, "cpu",
                               allocate_storage=False)
    assert only_window.can_hold([400, 400], 8) and not only_window.can_hold([400, 400, 400], 8)
    stateless = CacheManager([(StateNeed((3,)),)], (ScheduleEntry(0),), 4, 1, 2, torch.float32, "cpu",
                             allocate_storage=False)
    assert stateless.can_hold([10 ** 6, 10 ** 6], 64) and not stateless.can_hold([1, 1, 1], 64)   # slots alone
    # What it promises holds: a request stepped to its end in steps of at most 8 never holds more.
    m2 = CacheManager([(KVNeed(1, 4, window=10),)], (ScheduleEntry(0),), 4, 6, 1, torch.float32, "cpu",
                      allocate_storage=False)
    total = 0
    for n in (8, 8, 1, 1, 7, 8, 2, 8, 8, 8):
        total += n
        m2.reserve(["r"], [total])
        assert m2.groups[0].allocator.num_held <= m2.groups[0].pages_at(61, 8)
        m2.commit("r", total)
        m2.check_invariants()
