"""Host-side page bookkeeping: a pool of page numbers and per-request page tables.

A page holds ``page_size`` consecutive positions of one request.  The reference keeps
the same structure with 32-token pages, a LIFO free list and one table per sequence
slot (crates/thuban_model/src/pool.rs:11-118); it never returns pages that a sliding
window has passed.  Here each *group* of layers with the same needs owns a pool, and
a group with a window gives pages back as soon as no later query can reach them.
Nothing in this file touches a device.
"""
from __future__ import annotations

from ..errors import CacheError

NO_PAGE = -1


class PagePool:
    """Page numbers 0..n_pages-1 with a LIFO free list (a page just freed is the next
    one handed out, which keeps reuse frequent and easy to test)."""

    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise CacheError("a page pool needs at least one page")
        self.n_pages = int(n_pages)
        self._free = list(range(self.n_pages - 1, -1, -1))
        self._held = [False] * self.n_pages
        self.total_allocations = 0
        self.served = [0] * self.n_pages      # how many times each page was handed out

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def used_pages(self) -> int:
        return self.n_pages - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheError("page pool exhausted")
        p = self._free.pop()
        assert not self._held[p], f"page {p} handed out twice"
        self._held[p] = True
        self.total_allocations += 1
        self.served[p] += 1
        return p

    def give_back(self, page: int):
        if not (0 <= page < self.n_pages) or not self._held[page]:
            raise CacheError(f"page {page} freed twice or never allocated")
        self._held[page] = False
        self._free.append(page)

    def check(self):
        """Invariant: every page is either free exactly once or held."""
        assert len(set(self._free)) == len(self._free), "a page is on the free list twice"
        for p in range(self.n_pages):
            assert self._held[p] != (p in set(self._free)), f"page {p} both held and free (or neither)"


class PageTable:
    """Logical page index -> physical page for one request in one group.  Entries
    before ``first_live`` have been given back (window) and read NO_PAGE."""

    __slots__ = ("pages", "first_live")

    def __init__(self):
        self.pages: list[int] = []
        self.first_live = 0

    def held(self):
        return [p for p in self.pages if p != NO_PAGE]


class GroupPages:
    """Pages of one layer group: a pool plus one table per request slot."""

    def __init__(self, n_pages: int, page_size: int, window: int, max_slots: int, max_pages_per_request: int):
        self.page_size = int(page_size)
        self.window = int(window)          # 0 = every key is kept
        self.pool = PagePool(n_pages)
        self.tables = [PageTable() for _ in range(max_slots)]
        self.max_pages_per_request = int(max_pages_per_request)
        self.dirty_slots: set[int] = set()

    # the first position a query at ``pos`` can still see
    def first_visible(self, pos: int) -> int:
        return max(0, pos + 1 - self.window) if self.window else 0

    def pages_needed(self, slot: int, start: int, end: int) -> int:
        """New pages to run positions [start, end) of this request."""
        t = self.tables[slot]
        want_hi = -(-end // self.page_size)
        lo = max(len(t.pages), self.first_visible(start) // self.page_size)
        return max(0, want_hi - lo)

    def ensure(self, slot: int, start: int, end: int):
        """Make pages exist for positions [first_visible(start), end)."""
        t = self.tables[slot]
        want_hi = -(-end // self.page_size)
        if want_hi > self.max_pages_per_request:
            raise CacheError(f"context limit {self.max_pages_per_request * self.page_size} reached")
        need = self.pages_needed(slot, start, end)
        if need > self.pool.free_pages:
            raise CacheError(f"page pool exhausted: {need} pages requested, {self.pool.free_pages} free")
        first = self.first_visible(start) // self.page_size
        while len(t.pages) < want_hi:
            i = len(t.pages)
            if i < first:
                t.pages.append(NO_PAGE)       # never needed: behind the window from the start
                t.first_live = max(t.first_live, i + 1)
            else:
                t.pages.append(self.pool.take())
            self.dirty_slots.add(slot)

    def release_behind(self, slot: int, next_pos: int) -> int:
        """Give back pages that no query at ``next_pos`` or later can see."""
        if not self.window:
            return 0
        t = self.tables[slot]
        dead_hi = min(self.first_visible(next_pos) // self.page_size, len(t.pages))
        n = 0
        for i in range(t.first_live, dead_hi):
            if t.pages[i] != NO_PAGE:
                self.pool.give_back(t.pages[i])
                t.pages[i] = NO_PAGE
                n += 1
        if dead_hi > t.first_live:
            t.first_live = dead_hi
            self.dirty_slots.add(slot)
        return n

    def release_all(self, slot: int) -> int:
        t = self.tables[slot]
        held = t.held()
        for p in held:
            self.pool.give_back(p)
        t.pages = []
        t.first_live = 0
        self.dirty_slots.add(slot)
        return len(held)

    def truncate(self, slot: int, keep_tokens: int):
        """Drop pages above ``keep_tokens`` positions (crates/thuban_model/src/pool.rs:73-79)."""
        t = self.tables[slot]
        keep = min(-(-keep_tokens // self.page_size), len(t.pages))
        for p in t.pages[keep:]:
            if p != NO_PAGE:
                self.pool.give_back(p)
        del t.pages[keep:]
        t.first_live = min(t.first_live, keep)
        self.dirty_slots.add(slot)

    def check(self):
        self.pool.check()
        seen = set()
        for t in self.tables:
            for p in t.held():
                assert p not in seen, f"page {p} held by two requests"
                seen.add(p)
        assert len(seen) == self.pool.used_pages, "a page is lost (held by no request, not free)"
