"""Fixed-size pages of one cache group: a FIFO free list and reference counts.

The reference's PagedAllocator (engine/core/kv_cache.py:124-301) hands pages out from the
left of a deque and puts freed pages back at the right (:155-156, :252-261), so a freed page
is used again only after every page that was free before it.  The same order is kept here.
Page 0 is never handed out: block-table entries that point nowhere (padding, pages a window
has passed) hold 0, so every entry addresses memory that exists."""
from __future__ import annotations

from collections import deque


class PagePool:
    NULL_PAGE = 0

    def __init__(self, num_pages: int):
        if num_pages < 1:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages                       # usable pages: ids 1..num_pages
        self.free = deque(range(1, num_pages + 1))
        self.ref = [0] * (num_pages + 1)

    @property
    def num_free(self) -> int:
        return len(self.free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self.free)

    def take(self) -> int:
        if not self.free:
            raise RuntimeError("page pool is empty")
        page = self.free.popleft()
        assert self.ref[page] == 0, f"page {page} was free and referenced"
        self.ref[page] = 1
        return page

    def share(self, page: int) -> None:
        """One more holder of a page in use (kept for prefix sharing; unused by the engine)."""
        assert self.ref[page] > 0
        self.ref[page] += 1

    def give(self, page: int) -> None:
        if page == self.NULL_PAGE:
            raise ValueError("the null page is never freed")
        if self.ref[page] <= 0:
            raise RuntimeError(f"page {page} freed twice")
        self.ref[page] -= 1
        if self.ref[page] == 0:
            self.free.append(page)
