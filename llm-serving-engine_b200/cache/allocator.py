"""Page allocator: a FIFO free list with a use count per page.

First-in first-out reuse and the count per page follow src/llmserve/kv_cache.py:75-112. Pages are
not cleared when they are handed out again; readers never look past a request's own tokens.
"""

from __future__ import annotations

from collections import deque


class OutOfPages(RuntimeError):
    """No free page (or state slot) is left."""


class PageAllocator:
    def __init__(self, num_pages: int) -> None:
        if num_pages < 1:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self.free: deque[int] = deque(range(num_pages))
        self.ref = [0] * num_pages

    @property
    def num_free(self) -> int:
        return len(self.free)

    def allocate(self) -> int:
        if not self.free:
            raise OutOfPages("page pool exhausted")
        p = self.free.popleft()
        if self.ref[p] != 0:
            raise AssertionError(f"page {p} was on the free list while in use")
        self.ref[p] = 1
        return p

    def release(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise ValueError(f"page {page} is outside the pool")
        if self.ref[page] != 1:
            raise AssertionError(f"page {page} freed while its use count is {self.ref[page]}")
        self.ref[page] = 0
        self.free.append(page)

    def check_invariants(self) -> None:
        free = list(self.free)
        assert len(free) == len(set(free)), "a page is on the free list twice"
        for p in range(self.num_pages):
            assert self.ref[p] in (0, 1), f"page {p} has use count {self.ref[p]}"
        assert all(self.ref[p] == 0 for p in free), "a page in use is on the free list"
        assert sum(self.ref) + len(free) == self.num_pages, "a page is lost"
