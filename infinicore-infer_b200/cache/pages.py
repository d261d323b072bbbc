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
    def __init__(self, num_pages: int, reserved: int = 1, name: str = ""):
        if num_pages <= reserved:
            raise ValueError(f"a pool of {num_pages} pages with {reserved} reserved holds nothing")
        self.num_pages = num_pages
        self.reserved = reserved
        self.name = name
        # stack: pop from the end; lowest page first at the start
        self._free: List[int] = list(range(num_pages - 1, reserved - 1, -1))
        self._held = [False] * num_pages
        self.high_water = 0

    @property
    def capacity(self) -> int:
        return self.num_pages - self.reserved

    @property
    def available(self) -> int:
        return len(self._free)

    @property
    def in_use(self) -> int:
        return self.capacity - len(self._free)

    def alloc(self, n: int) -> List[int]:
        if n < 0:
            raise ValueError("negative page count")
        if n > len(self._free):
            raise OutOfPages(n, len(self._free), self.name)
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        self.high_water = max(self.high_water, self.in_use)
        return out

    def free(self, pages: Iterable[int]) -> None:
        pages = list(pages)
        for p in pages:
            if not (self.reserved <= p < self.num_pages):
                raise ValueError(f"page {p} is not one of this pool's")
            if not self._held[p]:
                raise ValueError(f"page {p} freed twice (or never handed out)")
        if len(set(pages)) != len(pages):
            raise ValueError("a page appears twice in one free")
        for p in pages:
            self._held[p] = False
            self._free.append(p)

    def held_pages(self) -> List[int]:
        return [p for p in range(self.reserved, self.num_pages) if self._held[p]]
