"""Cache groups: layers with the same needs share one pool and one block table per request.

A mixer says what it needs with a request record: ``PagedKV`` (keys and values in pages,
all of them or a window) or ``StateSlot`` (state of fixed size per request) or nothing.
Caches whose ``PagedKV`` records are equal form a group: they have pages of their own, a
block table per request that all caches of the group index with, and their own rule for
giving pages back (a window group frees the pages that every later query has passed).

The reference has one kind only, a whole-context tensor per layer and request
(src/models/jiuge/jiuge_kv_cache.cpp:3-23); pages, tables and groups have no counterpart.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np

from .pages import OutOfPages, PagePool

NO_PAGE = 0     # block-table entry of a block that holds nothing (the null page)


class CacheNeed:
    """What a mixer asks of the cache manager, as an object that knows how to provide it.  The manager and the
    scheduler call these methods and look at nothing else, so another kind of need (a class with the same methods,
    defined beside its mixer) is an addition, not a change:

    ``group_key()``              needs with equal keys share one group (a pool and block tables of their own); None: this
                                 need takes no pages and forms no group;
    ``make_group(...)``          the group's bookkeeping: an object with ``pages_needed / reserve / give_back / trim /
                                 truncate / release / row`` and a ``pool`` (see ``CacheGroup``);
    ``make_storage(...)``        device memory for the caches of a group (or for one cache without a group);
    ``make_view(...)``           what the mixer of one cache is handed at every step;
    ``most_pages_alone(...)``    pages that a request of ``total`` tokens holds at most when it runs alone with portions of
                                 ``chunk`` tokens (the scheduler's "can this request ever fit").
    """

    def group_key(self):
        return None

    def most_pages_alone(self, total: int, chunk: int, page_size: int) -> int:
        return 0


@dataclass(frozen=True)
class PagedKV(CacheNeed):
    """Keys and values of ``num_kv_heads`` heads of ``head_dim`` for every cached position."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None      # None: all keys are kept

    def group_key(self):
        return self

    def make_group(self, cache_ids, num_pages: int, page_size: int, max_blocks: int) -> "CacheGroup":
        return CacheGroup(self, cache_ids, num_pages, page_size, max_blocks=max_blocks)

    def make_storage(self, count: int, num_pages: int, page_size: int, num_slots: int, dtype, device):
        import torch
        if device is None:
            return None
        shape = (count, num_pages, self.num_kv_heads, page_size, self.head_dim)
        # zeros: what lies beyond a request's last position in a held page must be finite for every kernel
        return torch.zeros(shape, dtype=dtype, device=device), torch.zeros(shape, dtype=dtype, device=device)

    def make_view(self, storage, index: int, group_index: int, page_size: int):
        from .manager import KVView
        if storage is None:
            return KVView(group_index, None, None, page_size)
        return KVView(group_index, storage[0][index], storage[1][index], page_size)

    def most_pages_alone(self, total: int, chunk: int, page_size: int) -> int:
        span = total if self.window is None else min(total, self.window + chunk + page_size)
        return (span + page_size - 1) // page_size


@dataclass(frozen=True)
class StateSlot(CacheNeed):
    """Per-request state of fixed shape, e.g. a recurrent mixer's."""
    shape: Tuple[int, ...]
    dtype: str = "float32"

    def make_storage(self, count: int, num_pages: int, page_size: int, num_slots: int, dtype, device):
        import torch
        if device is None:
            return None
        return torch.zeros((num_slots,) + tuple(self.shape), dtype=getattr(torch, self.dtype), device=device)

    def make_view(self, storage, index: int, group_index: int, page_size: int):
        from .manager import StateView
        return StateView(storage)


class CacheGroup:
    """Host bookkeeping of one group: pool, block tables, trimming."""

    def __init__(self, need: PagedKV, cache_ids: List[int], num_pages: int, page_size: int, name: str = "",
                 max_blocks: Optional[int] = None):
        self.need = need
        self.cache_ids = list(cache_ids)
        self.page_size = page_size
        self.name = name or f"kv{need.num_kv_heads}x{need.head_dim}" + (f"w{need.window}" if need.window else "")
        self.pool = PagePool(num_pages, reserved=1, name=self.name)
        self.tables: Dict[object, List[int]] = {}      # request -> page of each block (NO_PAGE if none)
        self.first_block: Dict[object, int] = {}       # request -> first block still held
        # requests whose table may have a block without a page between first_block and its end; for all
        # others the blocks a step lacks are simply those beyond the table's end (no scan)
        self._holes: set = set()
        # with `max_blocks`: every table also as an int32 row, kept in step with the list, so that a step
        # copies a request's row into its upload buffer in one piece
        self.max_blocks = max_blocks
        self.rows: Dict[object, np.ndarray] = {}

    # -- how many new pages a request needs to hold positions [first_needed, new_len) -------
    def _first_needed_block(self, start: int) -> int:
        """First block that queries at positions >= start can still see."""
        if self.need.window is None:
            return 0
        return max(0, start - self.need.window + 1) // self.page_size

    def pages_needed(self, req, start: int, new_len: int) -> int:
        table = self.tables.get(req, [])
        last = (new_len + self.page_size - 1) // self.page_size
        first = max(self._first_needed_block(start), self.first_block.get(req, 0))
        if req not in self._holes and first <= len(table):
            return max(0, last - len(table))
        return sum(1 for b in range(first, last) if b >= len(table) or table[b] == NO_PAGE)

    def reserve(self, req, start: int, new_len: int) -> List[int]:
        """Make sure pages exist for positions that a step over [start, new_len) touches."""
        table = self.tables.setdefault(req, [])
        self.first_block.setdefault(req, 0)
        last = (new_len + self.page_size - 1) // self.page_size
        first = max(self._first_needed_block(start), self.first_block[req])
        if req not in self._holes and first <= len(table):
            want = list(range(len(table), last))
        else:
            want = [b for b in range(first, last) if b >= len(table) or table[b] == NO_PAGE]
        pages = self.pool.alloc(len(want))           # raises OutOfPages before anything changes
        if first > len(table):
            self._holes.add(req)                     # blocks between the table's end and `first` stay empty
        while len(table) < last:
            table.append(NO_PAGE)
        for b, p in zip(want, pages):
            table[b] = p
        if self.max_blocks is not None and want:
            row = self.rows.get(req)
            if row is None:
                row = self.rows[req] = np.zeros(self.max_blocks, dtype=np.int32)
            row[want] = pages
        return pages

    def give_back(self, req, pages: List[int]) -> None:
        """Undo a ``reserve`` (used when another group of the same step ran out)."""
        table = self.tables[req]
        back = set(pages)
        for b, p in enumerate(table):
            if p in back:
                table[b] = NO_PAGE
                if req in self.rows:
                    self.rows[req][b] = NO_PAGE
        while table and table[-1] == NO_PAGE and len(table) > self.first_block.get(req, 0):
            table.pop()                              # what was reserved last lies at the end
        if any(p == NO_PAGE for p in table[self.first_block.get(req, 0):]):
            self._holes.add(req)
        self.pool.free(pages)

    def trim(self, req, new_len: int) -> int:
        """Free the pages that no query at a position >= new_len can see.  Returns the count."""
        if self.need.window is None or req not in self.tables:
            return 0
        table = self.tables[req]
        keep_from = self._first_needed_block(new_len)
        freed = []
        for b in range(self.first_block[req], min(keep_from, len(table))):
            if table[b] != NO_PAGE:
                freed.append(table[b])
                table[b] = NO_PAGE
                if req in self.rows:
                    self.rows[req][b] = NO_PAGE
        self.first_block[req] = max(self.first_block[req], min(keep_from, len(table)))
        self.pool.free(freed)
        return len(freed)

    def truncate(self, req, new_len: int) -> int:
        """Drop what lies at positions >= new_len (a request that goes back to a shared prefix)."""
        table = self.tables.get(req)
        if table is None:
            return 0
        keep = (new_len + self.page_size - 1) // self.page_size
        if self.need.window is not None and self._first_needed_block(new_len) < self.first_block.get(req, 0):
            raise ValueError(f"cache group {self.name}: positions before {new_len} have left the window already")
        freed = [p for p in table[keep:] if p != NO_PAGE]
        del table[keep:]
        if req in self.rows:
            self.rows[req][keep:] = NO_PAGE
        self.pool.free(freed)
        return len(freed)

    def release(self, req) -> int:
        table = self.tables.pop(req, None)
        self.first_block.pop(req, None)
        self._holes.discard(req)
        self.rows.pop(req, None)
        if table is None:
            return 0
        pages = [p for p in table if p != NO_PAGE]
        self.pool.free(pages)
        return len(pages)

    def table(self, req) -> List[int]:
        return self.tables.get(req, [])

    def row(self, req) -> Optional[np.ndarray]:
        """The table as an int32 row of ``max_blocks`` entries (None if the request holds nothing yet)."""
        return self.rows.get(req)
