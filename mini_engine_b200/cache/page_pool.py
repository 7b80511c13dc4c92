"""Pages of one cache group: free list, reference counts, content hashes.

Reference bookkeeping (engine/block_manager.py:6-66): a free deque from whose front fresh
pages are taken and to whose back released pages go, a used set, reference counts, and a
hash per page that survives the release so that a freed page can still be found as a
prefix until it is taken for new content.
"""
from __future__ import annotations

from collections import deque


class PagePoolError(RuntimeError):
    pass


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages < 1:
            raise PagePoolError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self.ref_count = [0] * num_pages
        self.page_hash = [-1] * num_pages
        self.page_tokens: list[list[int]] = [[] for _ in range(num_pages)]
        self.hash_to_page: dict[int, int] = {}
        self.free: deque[int] = deque(range(num_pages))
        self.used: set[int] = set()

    @property
    def num_free(self) -> int:
        return len(self.free)

    def take_fresh(self) -> int:
        """A page for new content: front of the free list; its old hash is forgotten."""
        if not self.free:
            raise PagePoolError("no free page")
        page = self.free.popleft()
        if self.ref_count[page] != 0:
            raise PagePoolError(f"page {page} is on the free list but has {self.ref_count[page]} holders")
        h = self.page_hash[page]
        if h != -1 and self.hash_to_page.get(h) == page:
            del self.hash_to_page[h]
        self.page_hash[page] = -1
        self.page_tokens[page] = []
        self.ref_count[page] = 1
        self.used.add(page)
        return page

    def share(self, page: int) -> None:
        """One more holder of a page that already has content (a prefix hit)."""
        if self.ref_count[page] == 0:
            self.free.remove(page)          # still hashed, sitting on the free list
            self.used.add(page)
        self.ref_count[page] += 1

    def release(self, page: int) -> None:
        if self.ref_count[page] <= 0:
            raise PagePoolError(f"page {page} is released but has no holder")
        self.ref_count[page] -= 1
        if self.ref_count[page] == 0:
            self.used.remove(page)
            self.free.append(page)

    def set_hash(self, page: int, h: int, tokens: list[int]) -> None:
        self.page_hash[page] = h
        self.page_tokens[page] = tokens
        self.hash_to_page[h] = page

    def lookup(self, h: int, tokens: list[int]) -> int:
        page = self.hash_to_page.get(h, -1)
        if page == -1 or self.page_tokens[page] != tokens:     # collision check
            return -1
        return page

    def check(self) -> None:
        """Invariants: every page is free or used, never both; counts agree."""
        free = list(self.free)
        if len(set(free)) != len(free):
            raise PagePoolError("a page is on the free list twice")
        if set(free) & self.used:
            raise PagePoolError("a page is both free and used")
        if len(free) + len(self.used) != self.num_pages:
            raise PagePoolError("a page is lost")
        for p in range(self.num_pages):
            if (self.ref_count[p] > 0) != (p in self.used):
                raise PagePoolError(f"page {p}: holders and used set disagree")
