"""The cache manager: paged keys and values per layer group, block tables per request,
and slots for per-request state of fixed size.

Layer calls with the same needs (number of KV heads, head size, window) form a group;
a group has a page pool and block tables of its own, and every call in it has its own
storage indexed by the group's page numbers.  Beside the pages, each call that
declares fixed-size state gets one slab ``[max_slots, *shape]`` that is zeroed when a
request is admitted; the reference keeps such state outside its paged pool, indexed
by sequence slot, in the same way (crates/thuban_architectures/src/qwen35/state.rs:5-55).
Phi-MoE has one group and no state.

The bookkeeping (free lists, tables, which slot is live) is done by the native runtime
(``csrc/host/runtime.cpp``), which also keeps the host mirror of each block table up to date;
this file owns the device memory and copies changed table rows to it.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..csrc import runtime as rt
from ..errors import CacheError
from .pages import NO_PAGE, GroupPages


@dataclass(frozen=True)
class KVSpec:
    """What a mixer needs cached per token: ``num_kv_heads`` keys of ``head_dim`` numbers and as many values of
    ``value_dim`` numbers (default: as wide as the keys; 0: keys only).  ``window`` 0 means every key stays
    reachable; otherwise only the last ``window`` positions."""
    num_kv_heads: int
    head_dim: int
    window: int = 0
    value_dim: int | None = None

    @property
    def value_width(self) -> int:
        return self.head_dim if self.value_dim is None else int(self.value_dim)


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size state a mixer keeps per request (shape without the slot axis)."""
    shape: tuple
    dtype: torch.dtype = torch.float32


class GroupCache:
    """Device side of one group: K/V storage for each of its calls and the block table."""

    def __init__(self, spec: KVSpec, calls, n_pages: int, page_size: int, max_slots: int, max_pages_per_request: int,
                 dtype, device):
        self.spec = spec
        self.calls = list(calls)
        # the host mirror of the block table is written by the native bookkeeping
        self._host_table = torch.full((max_slots, max_pages_per_request), NO_PAGE, dtype=torch.int32)
        if torch.device(device).type == "cuda":
            self._host_table = self._host_table.pin_memory()
        pages = GroupPages(n_pages, page_size, spec.window, max_slots, max_pages_per_request,
                           host_table_ptr=self._host_table.data_ptr())
        self.pages = pages
        P = pages.page_size
        n = pages.pool.n_pages
        # keys [call, page, kv_head, position in page, head_dim] and values [..., value width]: one page of one
        # head is a contiguous P x width tile; keys and values may differ in width
        self.keys = torch.zeros((len(self.calls), n, spec.num_kv_heads, P, spec.head_dim), dtype=dtype, device=device)
        self.values = torch.zeros((len(self.calls), n, spec.num_kv_heads, P, spec.value_width), dtype=dtype, device=device)
        self.block_table = torch.full((max_slots, max_pages_per_request), NO_PAGE, dtype=torch.int32, device=device)
        # The copy to the device is asynchronous and may run long after it was asked for (behind a whole step
        # that is still running), while the bookkeeping goes on changing the host mirror for the next step:
        # the changed rows are therefore copied from a snapshot, two of which alternate.
        self._cuda = torch.device(device).type == "cuda"
        if self._cuda:
            self._snapshots = [torch.empty_like(self._host_table).pin_memory() for _ in range(2)]
            self._snapshot_sent = [torch.cuda.Event(), torch.cuda.Event()]
            self._snapshot_used = [False, False]
            self._next_snapshot = 0

    def sync_tables(self):
        """Copy the rows of changed block tables to the device."""
        lo, hi = self.pages.take_dirty()
        if lo >= hi:
            return
        if not self._cuda:
            self.block_table[lo:hi].copy_(self._host_table[lo:hi])
            return
        i = self._next_snapshot
        self._next_snapshot ^= 1
        if self._snapshot_used[i]:
            self._snapshot_sent[i].synchronize()      # its last copy has left it (two syncs ago: long done)
        snap = self._snapshots[i]
        snap[lo:hi].copy_(self._host_table[lo:hi])
        self.block_table[lo:hi].copy_(snap[lo:hi], non_blocking=True)
        self._snapshot_sent[i].record()
        self._snapshot_used[i] = True

    def view(self, call_index: int):
        i = self.calls.index(call_index)
        return CacheView(self.keys[i], self.values[i], self.block_table, self.pages.page_size, self.spec)


@dataclass
class CacheView:
    """What a mixer call sees of the cache: its K pages [page, kv_head, P, head_dim], its V pages
    [page, kv_head, P, value width] and its group's block table [slot, logical page]."""
    k: torch.Tensor
    v: torch.Tensor
    block_table: torch.Tensor
    page_size: int
    spec: KVSpec


class CacheManager:
    """Slots, pages and state for all requests of one model.

    ``kv_calls``: call index -> KVSpec for calls that own a cache.
    ``state_calls``: call index -> StateSpec for calls with fixed-size state.
    """

    def __init__(self, kv_calls: dict, state_calls: dict, *, page_size: int, n_pages: int,
                 max_slots: int, max_context: int, dtype, device):
        if page_size <= 0 or page_size % 16:
            raise CacheError(f"page_size must be a positive multiple of 16, got {page_size}")
        self.page_size = int(page_size)
        self.max_slots = int(max_slots)
        self.max_context = int(max_context)
        self.device = device
        max_pages_per_request = -(-max_context // page_size)
        by_spec: dict = {}
        for call, spec in kv_calls.items():
            by_spec.setdefault(spec, []).append(call)
        self._lib = rt.lib()
        self._core = self._lib.flint_rt_cache_create(self.page_size, self.max_slots, self.max_context)
        self.groups: list[GroupCache] = []
        self._group_of_call = {}
        for spec, calls in by_spec.items():
            g = GroupCache(spec, calls, n_pages, page_size, max_slots, max_pages_per_request, dtype, device)
            self._lib.flint_rt_cache_add_group(self._core, g.pages.handle)
            for c in calls:
                self._group_of_call[c] = g
            self.groups.append(g)
        self.state = {call: torch.zeros((max_slots, *spec.shape), dtype=spec.dtype, device=device)
                      for call, spec in state_calls.items()}

    def __del__(self):
        if getattr(self, "_core", None):
            self._lib.flint_rt_cache_destroy(self._core)
            self._core = None

    @property
    def core(self):
        """Handle of the native bookkeeping (for the native scheduler)."""
        return self._core

    # ------------------------------------------------------------------ slots
    @property
    def free_slots(self) -> int:
        return self._lib.flint_rt_cache_free_slots(self._core)

    def admit(self) -> int:
        """Take a slot for a new request and zero its state."""
        slot = rt.checked(self._lib.flint_rt_cache_admit(self._core))
        self.reset_state(slot)
        return slot

    def reset_state(self, slot: int):
        for s in self.state.values():
            s[slot].zero_()

    def release(self, slot: int):
        """Give back the slot and every page it holds."""
        rt.checked(self._lib.flint_rt_cache_release(self._core, int(slot)))

    # ------------------------------------------------------------------ pages
    def pages_needed(self, slot: int, start: int, end: int) -> int:
        """The largest number of new pages any group needs to run positions [start, end)."""
        return self._lib.flint_rt_cache_pages_needed(self._core, slot, start, end)

    def free_pages(self) -> int:
        return self._lib.flint_rt_cache_free_pages(self._core)

    def can_run(self, slot: int, start: int, end: int) -> bool:
        return bool(self._lib.flint_rt_cache_can_run(self._core, slot, start, end))

    def ensure(self, slot: int, start: int, end: int):
        """Make pages cover what running positions [start, end) reads and writes."""
        rt.checked(self._lib.flint_rt_cache_ensure(self._core, int(slot), int(start), int(end)))

    def advance(self, slot: int, next_pos: int):
        """After a step: positions below the windows of all later queries are given back."""
        rt.checked(self._lib.flint_rt_cache_advance(self._core, int(slot), int(next_pos)))

    def sync(self):
        for g in self.groups:
            g.sync_tables()

    def view(self, call_index: int) -> CacheView | None:
        g = self._group_of_call.get(call_index)
        return g.view(call_index) if g is not None else None

    def state_of(self, call_index: int):
        return self.state.get(call_index)

    def check(self):
        rt.checked(self._lib.flint_rt_cache_check(self._core))
