"""Host-side page bookkeeping: a pool of page numbers and per-request page tables.

A page holds ``page_size`` consecutive positions of one request.  The reference keeps
the same structure with 32-token pages, a LIFO free list and one table per sequence
slot (crates/thuban_model/src/pool.rs:11-118); it never returns pages that a sliding
window has passed.  Here each *group* of layers with the same needs owns a pool, and
a group with a window gives pages back as soon as no later query can reach them.

The bookkeeping itself lives in the native runtime (``csrc/host/runtime.cpp``); the classes
here are its Python faces.  Nothing in this file touches a device.
"""
from __future__ import annotations

from ctypes import c_int, byref

from ..csrc import runtime as rt
from ..errors import CacheError

NO_PAGE = -1


class _Native:
    """Owner of one native group (pool + tables)."""

    def __init__(self, n_pages, page_size, window, max_slots, max_pages_per_request, host_table_ptr=None):
        self.lib = rt.lib()
        self.handle = self.lib.flint_rt_group_create(n_pages, page_size, window, max_slots, max_pages_per_request,
                                                     host_table_ptr)
        if not self.handle:
            raise CacheError((self.lib.flint_rt_last_error() or b"cannot create a page pool").decode())

    def __del__(self):
        if getattr(self, "handle", None):
            self.lib.flint_rt_group_destroy(self.handle)
            self.handle = None


class PagePool:
    """Page numbers 0..n_pages-1 with a LIFO free list (a page just freed is the next
    one handed out, which keeps reuse frequent and easy to test)."""

    def __init__(self, n_pages: int, _native: _Native | None = None):
        if n_pages <= 0:
            raise CacheError("a page pool needs at least one page")
        self.n_pages = int(n_pages)
        self._n = _native or _Native(self.n_pages, 1, 0, 1, 1)
        self._lib = self._n.lib

    @property
    def free_pages(self) -> int:
        return self._lib.flint_rt_group_free_pages(self._n.handle)

    @property
    def used_pages(self) -> int:
        return self.n_pages - self.free_pages

    @property
    def total_allocations(self) -> int:
        return self._lib.flint_rt_group_total_allocations(self._n.handle)

    @property
    def served(self) -> list:
        """How many times each page was handed out."""
        out = (c_int * self.n_pages)()
        self._lib.flint_rt_group_served(self._n.handle, out)
        return list(out)

    def take(self) -> int:
        return rt.checked(self._lib.flint_rt_group_take(self._n.handle))

    def give_back(self, page: int):
        rt.checked(self._lib.flint_rt_group_give_back(self._n.handle, int(page)))

    def check(self):
        """Invariant: every page is either free exactly once or held."""
        rt.checked(self._lib.flint_rt_group_check(self._n.handle, 0))


class PageTable:
    """Logical page index -> physical page for one request in one group (a read-only view of
    the native table).  Entries before ``first_live`` have been given back (window) and read
    NO_PAGE."""

    __slots__ = ("_n", "_slot", "_cap")

    def __init__(self, native: _Native, slot: int, cap: int):
        self._n, self._slot, self._cap = native, slot, cap

    @property
    def pages(self) -> list:
        out = (c_int * self._cap)()
        n = self._n.lib.flint_rt_group_table(self._n.handle, self._slot, out, self._cap)
        return list(out[:n])

    @property
    def first_live(self) -> int:
        return self._n.lib.flint_rt_group_first_live(self._n.handle, self._slot)

    def held(self):
        return [p for p in self.pages if p != NO_PAGE]


class GroupPages:
    """Pages of one layer group: a pool plus one table per request slot.  ``host_table_ptr``,
    if given, is the address of an int32 [max_slots, max_pages_per_request] array that mirrors
    the tables (the block table that is copied to the device)."""

    def __init__(self, n_pages: int, page_size: int, window: int, max_slots: int, max_pages_per_request: int,
                 host_table_ptr=None):
        self.page_size = int(page_size)
        self.window = int(window)          # 0 = every key is kept
        self.max_pages_per_request = int(max_pages_per_request)
        self._n = _Native(int(n_pages), self.page_size, self.window, int(max_slots), self.max_pages_per_request,
                          host_table_ptr)
        self._lib = self._n.lib
        self.pool = PagePool(n_pages, self._n)
        self.tables = [PageTable(self._n, s, self.max_pages_per_request) for s in range(max_slots)]

    @property
    def handle(self):
        return self._n.handle

    # the first position a query at ``pos`` can still see
    def first_visible(self, pos: int) -> int:
        return max(0, pos + 1 - self.window) if self.window else 0

    def pages_needed(self, slot: int, start: int, end: int) -> int:
        """New pages to run positions [start, end) of this request."""
        return self._lib.flint_rt_group_pages_needed(self._n.handle, slot, start, end)

    def ensure(self, slot: int, start: int, end: int):
        """Make pages exist for positions [first_visible(start), end)."""
        rt.checked(self._lib.flint_rt_group_ensure(self._n.handle, slot, start, end))

    def release_behind(self, slot: int, next_pos: int) -> int:
        """Give back pages that no query at ``next_pos`` or later can see."""
        return rt.checked(self._lib.flint_rt_group_release_behind(self._n.handle, slot, next_pos))

    def release_all(self, slot: int) -> int:
        return rt.checked(self._lib.flint_rt_group_release_all(self._n.handle, slot))

    def truncate(self, slot: int, keep_tokens: int):
        """Drop pages above ``keep_tokens`` positions (crates/thuban_model/src/pool.rs:73-79)."""
        rt.checked(self._lib.flint_rt_group_truncate(self._n.handle, slot, keep_tokens))

    def take_dirty(self):
        """(lo, hi): the range of slots whose tables changed since the last call; lo >= hi if none."""
        lo, hi = c_int(), c_int()
        self._lib.flint_rt_group_take_dirty(self._n.handle, byref(lo), byref(hi))
        return lo.value, hi.value

    def check(self):
        """The pool's invariant, and: no page is held by two requests, none is lost."""
        rt.checked(self._lib.flint_rt_group_check(self._n.handle, 1))
