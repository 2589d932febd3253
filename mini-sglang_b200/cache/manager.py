"""The cache manager: keys and values in pages with one block table per request and group,
and slots for per-request state of fixed size.

What a mixer keeps between steps is declared as a *need*:
  PagedKVNeed(n_kv_heads, head_dim, window)  keys and values of every token (window=None) or of
                                             the last `window` tokens only
  StateNeed(shape, dtype)                    an array of fixed size per request
Caches whose needs differ in kind (all keys / a window of them) form groups with pages of their
own: a page id of a group indexes the K and V arrays of every cache in that group, and each
group has its own pool and its own block table per request.  A request owns one slot (a row in
every block table and in every state array) from `open` to `close`.

    slot = mgr.open()                 take a request slot (state rows are zeroed)
    mgr.reserve(slot, n)              pages for the next n tokens in every group (all or nothing)
    mgr.slot_mapping(g, slot, s, n)   token slots (page * P + offset) of positions s..s+n-1
    mgr.commit(slot, n)               the n tokens are in the cache; pages a window has passed
                                      are given back
    mgr.close(slot)                   everything the request holds is given back

Pages are given back when a request ends or a window has passed them, and are handed out again
first-in first-out.  The reference's counterparts: mini_sglang/mem_cache/token2kv.py (pool and
allocator, one group), mini_sglang/mem_cache/req2token.py (request slots and block table).
"""

from __future__ import annotations

import dataclasses
from collections import deque
from typing import Dict, List, Optional, Sequence, Tuple, Union

import numpy as np

from .pages import OutOfPages, PagePool


@dataclasses.dataclass(frozen=True)
class PagedKVNeed:
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    q_heads: int = 0                 # hint for work splitting only


@dataclasses.dataclass(frozen=True)
class StateNeed:
    shape: Tuple[int, ...]
    dtype: str = "float32"           # "float32", "compute" (the engine's activation dtype) or "int32"


class OutOfSlots(RuntimeError):
    pass


class KVGroup:
    """Caches with the same kind of need: one pool, one block table per request."""

    def __init__(self, window: Optional[int], num_pages: int, max_reqs: int, max_pages_per_req: int):
        self.window = window
        self.pool = PagePool(num_pages)
        self.table = np.zeros((max_reqs + 1, max_pages_per_req), dtype=np.int32)
        self.n_pages = np.zeros(max_reqs + 1, dtype=np.int64)      # table entries in use (released ones included)
        self.first_live = np.zeros(max_reqs + 1, dtype=np.int64)   # entries below this were given back
        self.cache_ids: List[int] = []
        self.dirty: set = set()        # slots whose table row changed since a device copy of the table was last brought up to date


class CacheManager:
    def __init__(self, needs: Dict[int, Union[PagedKVNeed, StateNeed]], *, page_size: int, num_pages: int,
                 max_reqs: int, max_context_len: int, max_step_tokens: int = 0):
        if page_size < 1:
            raise ValueError("page_size must be at least 1")
        self.page_size = page_size
        self.max_reqs = max_reqs
        self.max_context_len = max_context_len
        self.max_pages_per_req = -(-max_context_len // page_size)
        self.needs = dict(needs)
        self.groups: List[KVGroup] = []
        self.group_of_cache: Dict[int, int] = {}
        by_window: Dict[Optional[int], int] = {}
        for cid in sorted(needs):
            need = needs[cid]
            if isinstance(need, PagedKVNeed):
                if need.window is not None and need.window < 1:
                    raise ValueError("a window must be at least 1 token")
                if need.window not in by_window:
                    n = num_pages
                    if need.window is not None:
                        per_req = -(-(need.window + max(max_step_tokens, 1)) // page_size) + 2
                        n = min(num_pages, max_reqs * per_req)
                    by_window[need.window] = len(self.groups)
                    self.groups.append(KVGroup(need.window, n, max_reqs, self.max_pages_per_req))
                g = by_window[need.window]
                self.groups[g].cache_ids.append(cid)
                self.group_of_cache[cid] = g
        self.state_ids = [cid for cid in sorted(needs) if isinstance(needs[cid], StateNeed)]
        self._free_slots = deque(range(1, max_reqs + 1))           # slot 0: dump row for padded batch rows
        self._open = np.zeros(max_reqs + 1, dtype=bool)
        self.length = np.zeros(max_reqs + 1, dtype=np.int64)       # tokens committed
        self.reserved = np.zeros(max_reqs + 1, dtype=np.int64)     # tokens with pages (>= length)
        self.borrowed = np.zeros(max_reqs + 1, dtype=np.int64)     # leading pages of group 0 owned by a prefix tree
        self.on_open = []                                          # callbacks(slot): zero state rows on the device

    # -- slots -------------------------------------------------------------------------
    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def open(self) -> int:
        if not self._free_slots:
            raise OutOfSlots(f"all {self.max_reqs} request slots are taken")
        slot = self._free_slots.popleft()
        self._open[slot] = True
        self.length[slot] = 0
        self.reserved[slot] = 0
        self.borrowed[slot] = 0
        for g in self.groups:
            g.n_pages[slot] = 0
            g.first_live[slot] = 0
        for cb in self.on_open:
            cb(slot)
        return slot

    def is_open(self, slot: int) -> bool:
        return bool(self._open[slot])

    # -- pages -------------------------------------------------------------------------
    def pages_needed(self, slot: int, n_new: int) -> List[int]:
        """New pages per group that `reserve(slot, n_new)` would take."""
        P = self.page_size
        total = int(self.reserved[slot]) + n_new if n_new > 0 else int(self.reserved[slot])
        return [max(0, -(-total // P) - int(g.n_pages[slot])) for g in self.groups]

    def reserve(self, slot: int, n_new: int) -> None:
        if not self._open[slot]:
            raise ValueError(f"slot {slot} is not open")
        total = int(self.reserved[slot]) + n_new
        if total > self.max_context_len:
            raise ValueError(f"request would hold {total} tokens, the context limit is {self.max_context_len}")
        need = self.pages_needed(slot, n_new)
        for g, n in zip(self.groups, need):
            if n > g.pool.available:
                raise OutOfPages(f"{n} pages wanted, {g.pool.available} free of {g.pool.num_pages}"
                                 + (f" (window {g.window})" if g.window else ""))
        for g, n in zip(self.groups, need):
            if n:
                k = int(g.n_pages[slot])
                g.table[slot, k:k + n] = g.pool.alloc(n)
                g.n_pages[slot] = k + n
                g.dirty.add(slot)
        self.reserved[slot] = total

    def adopt_prefix(self, slot: int, pages: Sequence[int]) -> None:
        """Start a fresh request on pages that a prefix tree owns (group 0, whole pages)."""
        if self.length[slot] or self.reserved[slot]:
            raise ValueError("a prefix can only be adopted by a request that holds nothing")
        if len(self.groups) != 1 or self.groups[0].window is not None or self.state_ids:
            raise ValueError("prefix reuse needs a single group that keeps all keys and no per-request state")
        g = self.groups[0]
        n = len(pages)
        g.table[slot, :n] = pages
        g.n_pages[slot] = n
        g.dirty.add(slot)
        self.borrowed[slot] = n
        self.length[slot] = self.reserved[slot] = n * self.page_size

    def replace_prefix(self, slot: int, table: Sequence[int], n_borrowed: int) -> None:
        """After a prefix tree took (or already had) the request's leading pages."""
        g = self.groups[0]
        g.table[slot, :len(table)] = table
        g.dirty.add(slot)
        self.borrowed[slot] = n_borrowed

    def slot_mapping(self, group: int, slot: int, start: int, n: int) -> np.ndarray:
        P = self.page_size
        pos = np.arange(start, start + n, dtype=np.int64)
        return (self.groups[group].table[slot, pos // P].astype(np.int64) * P + pos % P).astype(np.int32)

    def take_dirty_rows(self, group: int) -> List[Tuple[int, np.ndarray]]:
        """(slot, its table row) of every open request whose row changed since the last call: what a device copy of the
        group's block tables has to be given to be up to date."""
        g = self.groups[group]
        out = [(slot, g.table[slot, :int(g.n_pages[slot])]) for slot in sorted(g.dirty) if g.n_pages[slot] > 0]
        g.dirty.clear()
        return out

    def block_table_row(self, group: int, slot: int) -> np.ndarray:
        g = self.groups[group]
        return g.table[slot, :int(g.n_pages[slot])]

    def commit(self, slot: int, n_new: int) -> None:
        new_len = int(self.length[slot]) + n_new
        if new_len > self.reserved[slot]:
            raise ValueError("commit beyond the reserved pages")
        self.length[slot] = new_len
        P = self.page_size
        for g in self.groups:
            if g.window is None:
                continue
            dead = max(0, (new_len - g.window + 1) // P)       # pages wholly before the next query's window
            dead = min(dead, int(g.n_pages[slot]))
            first = int(g.first_live[slot])
            if dead > first:
                g.pool.free(int(p) for p in g.table[slot, first:dead])
                g.table[slot, first:dead] = 0
                g.first_live[slot] = dead
                g.dirty.add(slot)

    def owned_pages(self, slot: int, group: int = 0) -> List[int]:
        g = self.groups[group]
        lo = max(int(g.first_live[slot]), int(self.borrowed[slot]) if group == 0 else 0)
        return [int(p) for p in g.table[slot, lo:int(g.n_pages[slot])]]

    def close(self, slot: int, keep_pages: int = 0) -> None:
        """Give back the slot and every page the request owns; `keep_pages` leading owned pages of
        group 0 are left alone (a prefix tree took them)."""
        if not self._open[slot]:
            raise ValueError(f"slot {slot} closed twice")
        for gi, g in enumerate(self.groups):
            lo = int(g.first_live[slot])
            if gi == 0:
                lo = max(lo, int(self.borrowed[slot]) + keep_pages)
            hi = int(g.n_pages[slot])
            if hi > lo:
                g.pool.free(int(p) for p in g.table[slot, lo:hi])
            g.table[slot, :hi] = 0
            g.n_pages[slot] = 0
            g.first_live[slot] = 0
            g.dirty.discard(slot)
        self.length[slot] = self.reserved[slot] = self.borrowed[slot] = 0
        self._open[slot] = False
        self._free_slots.append(slot)

    # -- accounting --------------------------------------------------------------------
    def available_pages(self, group: int = 0) -> int:
        return self.groups[group].pool.available

    def check_idle(self, tree_pages: int = 0) -> None:
        """With no request open: every slot free and every page free or in the prefix tree."""
        if len(self._free_slots) != self.max_reqs:
            raise RuntimeError(f"leak: {self.max_reqs - len(self._free_slots)} request slots still taken")
        for gi, g in enumerate(self.groups):
            held = g.pool.in_use - (tree_pages if gi == 0 else 0)
            if held:
                raise RuntimeError(f"leak: {held} pages of group {gi} are neither free nor cached")
