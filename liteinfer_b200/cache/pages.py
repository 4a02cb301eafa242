"""Page and slot allocators: pure host bookkeeping, no tensors.

liteinfer/cache/block_pool.py:63-96 keeps a Python free list (`allocate` pops,
`free` appends), so a page given back is the next one handed out.  The same
last-in-first-out order is kept here because it makes reuse immediate, which
is what the replay tests lean on.  Beyond the reference, every page's state is
tracked, so holding a page twice or freeing it twice raises instead of
corrupting a neighbour's context.
"""

from __future__ import annotations


class CacheExhaustedError(RuntimeError):
    """The cache cannot hold what a step asks for; nothing was allocated."""


class OutOfPagesError(CacheExhaustedError):
    pass


class OutOfStateSlotsError(CacheExhaustedError):
    pass


class PageAllocator:
    """`num_pages` pages, handed out last-freed-first."""

    def __init__(self, num_pages: int) -> None:
        if num_pages < 1:
            raise ValueError("num_pages must be >= 1")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))  # pop() hands out page 0 first
        self._held = [False] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.num_pages - len(self._free)

    def allocate(self, count: int) -> list[int]:
        """`count` pages, or OutOfPagesError with nothing taken."""
        if count < 0:
            raise ValueError("count must be >= 0")
        if count > len(self._free):
            raise OutOfPagesError(f"{count} pages wanted, {len(self._free)} of {self.num_pages} free")
        pages = [self._free.pop() for _ in range(count)]
        for page in pages:
            assert not self._held[page], f"page {page} handed out while held"
            self._held[page] = True
        return pages

    def free(self, pages) -> None:
        for page in pages:
            if not 0 <= page < self.num_pages:
                raise ValueError(f"page {page} does not exist")
            if not self._held[page]:
                raise ValueError(f"page {page} is freed but not held")
            self._held[page] = False
            self._free.append(page)

    def is_held(self, page: int) -> bool:
        return self._held[page]


class SlotAllocator(PageAllocator):
    """Fixed-size per-request state slots; the same bookkeeping as pages."""

    def allocate_one(self) -> int:
        try:
            return self.allocate(1)[0]
        except OutOfPagesError as error:
            raise OutOfStateSlotsError(f"all {self.num_pages} state slots are taken") from error
