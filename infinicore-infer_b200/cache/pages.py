"""Page pool: the free list behind one group of cache layers.

Host-side bookkeeping only.  Pages are handed out last-freed-first, so a page that a
finished request gave back is the next one to be used again.  The first ``reserved`` pages
are never handed out; page 0 is the null page that padded rows of a captured decode step
write to.
"""
from __future__ import annotations

from typing import Iterable, List


class OutOfPages(RuntimeError):
    """The pool cannot satisfy a request for pages; nothing was taken."""

    def __init__(self, wanted: int, available: int, group: str = ""):
        self.wanted, self.available, self.group = wanted, available, group
        super().__init__(f"cache group {group or '?'}: {wanted} pages wanted, {available} free")


class PagePool:
    """The free list of one cache group.  The bookkeeping itself (which pages are free, in which order they go out,
    which are held) is ``jk::PagePool`` of csrc/host_rules.h, the same class that the C interface's pool is; this
    wrapper gives it Python's errors and names."""

    def __init__(self, num_pages: int, reserved: int = 1, name: str = ""):
        if num_pages <= reserved:
            raise ValueError(f"a pool of {num_pages} pages with {reserved} reserved holds nothing")
        from ..kernels.host import NativePagePool
        self.num_pages = num_pages
        self.reserved = reserved
        self.name = name
        self._pool = NativePagePool(num_pages, reserved)
        # how many pages are free, counted here as well: every page goes out and comes back through this object, and a
        # step asks for the count far more often than it takes a page
        self._free = num_pages - reserved

    @property
    def capacity(self) -> int:
        return self.num_pages - self.reserved

    @property
    def available(self) -> int:
        return self._free

    @property
    def in_use(self) -> int:
        return self.capacity - self._free

    @property
    def high_water(self) -> int:
        return self._pool.high_water()

    def alloc(self, n: int) -> List[int]:
        if n < 0:
            raise ValueError("negative page count")
        if n == 0:
            return []
        out = self._pool.alloc(n) if n <= self._free else None
        if out is None:
            raise OutOfPages(n, self._free, self.name)
        self._free -= n
        return out

    def free(self, pages: Iterable[int]) -> None:
        pages = list(pages)
        if not pages:
            return
        rc = self._pool.free(pages)
        if rc == 1:
            bad = next(p for p in pages if not (self.reserved <= p < self.num_pages))
            raise ValueError(f"page {bad} is not one of this pool's")
        if rc == 2:
            bad = next(p for p in pages if not self._pool.is_held(p))
            raise ValueError(f"page {bad} freed twice (or never handed out)")
        if rc == 3:
            raise ValueError("a page appears twice in one free")
        self._free += len(pages)

    def held_pages(self) -> List[int]:
        return [p for p in range(self.reserved, self.num_pages) if self._pool.is_held(p)]
