"""The cache manager: pages of keys and values per group of layers, block tables per request, state slots.

What the model must remember between steps is declared by its parts
(`KVNeed`, `StateNeed`).  Stops of the schedule whose needs are equal form a
*group*: one pool tensor [stops, 2, pages, kv_heads, page_size, head_dim], one
page allocator, and one block table per request (logical block -> page, -1 once
given back).  A group that keeps every key never frees a page before the
request ends; a group with a window frees the pages that the window has passed
after each step.  Beside the groups, every request holds one slot of
fixed-size state for the mixers that declare a `StateNeed` (the slot exists
even when no layer uses it, so the step function always passes one).  A layer
may declare several needs of either kind (two mixers in one block, a mixer with
a short convolution tail and a recurrent state); each is found under its name.

The reference keeps one pool for all layers and frees only at release
(liteinfer/cache/kv_cache.py:129-174, block_pool.py:28-100); its rule that a
reservation raises before anything is allocated (kv_cache.py:145-169) holds
here across all groups at once.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from liteinfer_b200.cache.pages import CacheExhaustedError, OutOfPagesError, PageAllocator, SlotAllocator
from liteinfer_b200.parts.context import KVCacheView, KVNeed, LayerCache, StateNeed
from liteinfer_b200.parts.spec import ScheduleEntry

__all__ = ["CacheManager", "CacheExhaustedError", "OutOfPagesError", "KVGroup"]


def _cdiv(a: int, b: int) -> int:
    return -(-a // b)


@dataclass
class KVGroup:
    need: KVNeed
    holders: list[tuple[int, str]]       # (schedule stop, need's name) of every cache kept here, in order
    allocator: PageAllocator
    page_size: int
    pool: torch.Tensor | None = None     # [len(holders), 2, pages, kv_heads, page_size, head_dim]
    tables: dict[str, list[int]] = field(default_factory=dict)

    @property
    def stops(self) -> list[int]:
        """Schedule stops that keep a cache here, in order (a stop with two such needs appears twice)."""
        return [stop for stop, _ in self.holders]

    def bytes_per_page(self, element_size: int) -> int:
        return len(self.holders) * 2 * self.need.kv_heads * self.page_size * self.need.head_dim * element_size

    def pages_at(self, total: int, largest_step: int) -> int:
        """The most pages a request holds here at any time on its way to `total` tokens, when no step brings it
        more than `largest_step` of them: every block for a group that keeps all keys; for a group with a
        window, the blocks that the window still reaches at a step's start plus those the step writes."""
        every = _cdiv(total, self.page_size)
        if self.need.window is None:
            return every
        span = self.need.window - 1 + max(1, min(largest_step, total))
        return min(every, _cdiv(span, self.page_size) + 1)

    def first_needed_block(self, total: int) -> int:
        """First logical block a request holding `total` tokens can still read."""
        if self.need.window is None:
            return 0
        # The next query sits at position >= total and sees keys > position - window.
        return max(0, total - self.need.window + 1) // self.page_size

    def missing_blocks(self, request_id: str, old_total: int, new_total: int) -> list[int]:
        """Logical blocks that positions [old_total, new_total) touch and that hold no page yet."""
        if new_total <= old_total:
            return []
        table = self.tables.get(request_id, [])
        first, last = old_total // self.page_size, (new_total - 1) // self.page_size
        return [b for b in range(first, last + 1) if b >= len(table) or table[b] < 0]


class CacheManager:
    def __init__(self, layer_needs: list[tuple], schedule: tuple[ScheduleEntry, ...], page_size: int,
                 num_pages: int, max_requests: int, dtype: torch.dtype, device: torch.device | str,
                 allocate_storage: bool = True) -> None:
        if page_size < 1:
            raise ValueError("page_size must be >= 1")
        self.page_size, self.num_pages, self.max_requests = page_size, num_pages, max_requests
        self.dtype, self.device = dtype, torch.device(device)
        self.schedule = schedule
        self.groups: list[KVGroup] = []
        self._stop_kv: dict[int, dict[str, tuple[int, int]]] = {}     # owning stop -> name -> (group, index in group)
        self._stop_state: dict[int, dict[str, torch.Tensor | None]] = {}
        self.slots = SlotAllocator(max_requests)
        self._slot_of: dict[str, int] = {}
        self._length: dict[str, int] = {}
        self._state_tensors: list[torch.Tensor] = []
        self._table_version: dict[str, int] = {}            # changes whenever a block table of the request does
        self._versions = 0

        by_need: dict[KVNeed, KVGroup] = {}
        for stop, entry in enumerate(schedule):
            if entry.cache_of is not None:
                continue
            for need in layer_needs[entry.layer]:
                if isinstance(need, KVNeed):
                    mine = self._stop_kv.setdefault(stop, {})
                    if need.name in mine:
                        raise ValueError(f"layer {entry.layer} declares two KV needs named {need.name!r}; "
                                         "give each a name of its own")
                    group = by_need.get(need)
                    if group is None:
                        group = KVGroup(need, [], PageAllocator(num_pages), page_size)
                        by_need[need] = group
                        self.groups.append(group)
                    mine[need.name] = (self.groups.index(group), len(group.holders))
                    group.holders.append((stop, need.name))
                elif isinstance(need, StateNeed):
                    mine = self._stop_state.setdefault(stop, {})
                    if need.name in mine:
                        raise ValueError(f"layer {entry.layer} declares two state needs named {need.name!r}; "
                                         "give each a name of its own")
                    state_dtype = torch.float32 if need.kind == "f32" else dtype
                    state = None
                    if allocate_storage:
                        state = torch.zeros((max_requests, *need.shape), dtype=state_dtype, device=self.device)
                        self._state_tensors.append(state)
                    mine[need.name] = state
                else:
                    raise TypeError(f"unknown cache need {need!r}")
        if allocate_storage:
            for group in self.groups:
                group.pool = torch.zeros(
                    (len(group.holders), 2, num_pages, group.need.kv_heads, page_size, group.need.head_dim),
                    dtype=dtype, device=self.device)

    # ----------------------------------------------------------- sizes
    def bytes_per_page(self) -> int:
        """Bytes that one page index costs across all groups."""
        element = torch.empty((), dtype=self.dtype).element_size()
        return sum(g.bytes_per_page(element) for g in self.groups)

    @staticmethod
    def bytes_per_page_for(layer_needs: list[tuple], schedule, page_size: int, dtype: torch.dtype) -> int:
        probe = CacheManager(layer_needs, schedule, page_size, 1, 1, dtype, "cpu", allocate_storage=False)
        return probe.bytes_per_page()

    # ----------------------------------------------------------- requests
    def has(self, request_id: str) -> bool:
        return request_id in self._length

    def length(self, request_id: str) -> int:
        """Tokens of this request that the cache holds (0 for a request not seen yet)."""
        return self._length.get(request_id, 0)

    def state_slot(self, request_id: str) -> int:
        return self._slot_of[request_id]

    def table_version(self, request_id: str) -> int:
        """A number that is new whenever one of the request's block tables (or its state slot) has changed: a
        caller that kept a copy of the tables may keep it while the number stays."""
        return self._table_version[request_id]

    def _touch(self, request_id: str) -> None:
        self._versions += 1
        self._table_version[request_id] = self._versions

    @property
    def live_requests(self) -> list[str]:
        return list(self._length)

    def can_hold(self, final_totals: list[int], largest_step: int) -> bool:
        """Whether requests that grow to `final_totals` tokens, in steps of at most `largest_step` tokens each,
        fit into the cache all at once: every group's pages (a window bounds what a request holds there) and the
        state slots.  A model without pages is held by its slots alone."""
        if len(final_totals) > self.max_requests:
            return False
        return all(sum(group.pages_at(total, largest_step) for total in final_totals) <= group.allocator.num_pages
                   for group in self.groups)

    def pages_missing(self, request_ids: list[str], new_totals: list[int]) -> list[int]:
        """Per group, how many more pages the reservation would take."""
        wanted = [0] * len(self.groups)
        for request_id, total in zip(request_ids, new_totals, strict=True):
            old = self.length(request_id)
            for g, group in enumerate(self.groups):
                wanted[g] += len(group.missing_blocks(request_id, old, total))
        return wanted

    def reserve(self, request_ids: list[str], new_totals: list[int]) -> None:
        """Make room for every request to grow to its new total, or raise with nothing changed.

        A request seen for the first time also takes its state slot here.
        """
        if len(set(request_ids)) != len(request_ids):
            raise ValueError("a request appears twice in one reservation")
        # The common decode step: every request is known and grows by tokens that still fit its last page.
        page = self.page_size
        lengths = self._length
        if all(r in lengths and 0 < total - lengths[r] <= -lengths[r] % page for r, total in zip(request_ids, new_totals, strict=True)):
            return
        for request_id, total in zip(request_ids, new_totals, strict=True):
            if total < self.length(request_id):
                raise ValueError(f"{request_id} holds {self.length(request_id)} tokens and cannot shrink to {total}")
        wanted = self.pages_missing(request_ids, new_totals)
        for g, group in enumerate(self.groups):
            if wanted[g] > group.allocator.num_free:
                raise OutOfPagesError(
                    f"cache group {g} needs {wanted[g]} more pages, {group.allocator.num_free} of "
                    f"{group.allocator.num_pages} are free")
        newcomers = [r for r in request_ids if r not in self._length]
        if len(newcomers) > self.slots.num_free:
            raise CacheExhaustedError(
                f"{len(newcomers)} new requests but {self.slots.num_free} of {self.max_requests} state slots are free")
        for request_id in newcomers:
            slot = self.slots.allocate_one()
            self._slot_of[request_id] = slot
            self._length[request_id] = 0
            for state in self._state_tensors:
                state[slot].zero_()
            for group in self.groups:
                group.tables[request_id] = []
            self._touch(request_id)
        for request_id, total in zip(request_ids, new_totals, strict=True):
            old = self._length[request_id]
            for group in self.groups:
                blocks = group.missing_blocks(request_id, old, total)
                if not blocks:
                    continue
                self._touch(request_id)
                pages = group.allocator.allocate(len(blocks))
                table = group.tables[request_id]
                for block, page in zip(blocks, pages, strict=True):
                    while len(table) <= block:
                        table.append(-1)
                    table[block] = page

    def commit(self, request_id: str, new_total: int) -> None:
        """The step that wrote up to `new_total` succeeded: count it, and give back what a window has passed."""
        self._length[request_id] = new_total
        for group in self.groups:
            if group.need.window is None:
                continue
            table = group.tables[request_id]
            passed = min(group.first_needed_block(new_total), len(table))
            freed = [table[b] for b in range(passed) if table[b] >= 0]
            if not freed:
                continue
            for b in range(passed):
                table[b] = -1
            group.allocator.free(freed)
            self._touch(request_id)

    def rollback(self, request_ids: list[str]) -> None:
        """A step failed after its reservation: give back the pages beyond what each request holds."""
        for request_id in request_ids:
            if request_id not in self._length:
                continue
            held = self._length[request_id]
            if held == 0:
                self.release(request_id)
                continue
            keep = _cdiv(held, self.page_size)
            for group in self.groups:
                table = group.tables[request_id]
                group.allocator.free([p for p in table[keep:] if p >= 0])
                del table[keep:]
            self._touch(request_id)

    def release(self, request_id: str) -> None:
        """The request is over: all its pages and its state slot go back."""
        if request_id not in self._length:
            return
        for group in self.groups:
            table = group.tables.pop(request_id)
            group.allocator.free([p for p in table if p >= 0])
        self.slots.free([self._slot_of.pop(request_id)])
        del self._length[request_id]
        del self._table_version[request_id]

    # -------------------------------------------------------------- views
    def block_table(self, group: int, request_id: str) -> list[int]:
        return self.groups[group].tables[request_id]

    def layer_caches(self) -> list[LayerCache]:
        """One `LayerCache` per stop of the schedule, sharing storage where the schedule says so."""
        caches: list[LayerCache] = []
        for stop, entry in enumerate(self.schedule):
            owner = stop if entry.cache_of is None else entry.cache_of
            cache = LayerCache(read_only=entry.cache_of is not None)
            for name, (g, index) in self._stop_kv.get(owner, {}).items():
                group = self.groups[g]
                cache.kvs[name] = KVCacheView(group.pool[index, 0], group.pool[index, 1], g, self.page_size)
            cache.states.update(self._stop_state.get(owner, {}))
            caches.append(cache)
        return caches

    def check_invariants(self) -> None:
        """No page lost, none held twice: every held page is in exactly one table."""
        for g, group in enumerate(self.groups):
            seen: set[int] = set()
            for request_id, table in group.tables.items():
                for page in table:
                    if page < 0:
                        continue
                    assert page not in seen, f"group {g}: page {page} is in two tables"
                    assert group.allocator.is_held(page), f"group {g}: page {page} of {request_id} is not held"
                    seen.add(page)
            assert len(seen) == group.allocator.num_held, (
                f"group {g}: {group.allocator.num_held} pages held but {len(seen)} are in tables")
        assert sorted(self._slot_of.values()) == sorted(set(self._slot_of.values()))
        assert len(self._slot_of) == self.slots.num_held
