"""A pool of cache pages: ids, a first-in-first-out free list and ownership checks.

Semantics of ``BlockAllocator`` (inference_engine/block_manager.py:14-44): page 0 is a scratch
page that is never handed out (padding rows of a captured decode step read and write it),
pages are taken from the left of the free list and given back on the right, so a freed page
is used again only after the pages that were free before it.  Added here: the pool knows the
owner of every page and refuses to free a page that is not held, or to hand one out twice."""
from __future__ import annotations

from collections import deque


class PageError(RuntimeError):
    """A page was freed twice, freed without being held, or the pool ran dry."""


class PagePool:
    def __init__(self, num_pages: int, reserved: int = 1):
        if num_pages <= reserved:
            raise ValueError(f"a pool needs more than {reserved} page(s), got {num_pages}")
        self.num_pages = num_pages
        self.reserved = reserved
        self._free = deque(range(reserved, num_pages))
        self._held = [False] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_usable(self) -> int:
        return self.num_pages - self.reserved

    def can_take(self, n: int, watermark: int = 0) -> bool:
        return len(self._free) - n >= watermark

    def take(self, n: int) -> list[int]:
        if n > len(self._free):
            raise PageError(f"asked for {n} pages, {len(self._free)} free")
        out = [self._free.popleft() for _ in range(n)]
        for p in out:
            if self._held[p]:
                raise PageError(f"page {p} was on the free list while held")
            self._held[p] = True
        return out

    def give_back(self, pages) -> None:
        for p in pages:
            if not (self.reserved <= p < self.num_pages):
                raise PageError(f"page {p} is not a page of this pool")
            if not self._held[p]:
                raise PageError(f"page {p} freed twice or never taken")
            self._held[p] = False
            self._free.append(p)

    def held_pages(self) -> list[int]:
        return [p for p in range(self.num_pages) if self._held[p]]

    def check(self) -> None:
        """Every usable page is either free once or held, never both."""
        free = list(self._free)
        if len(set(free)) != len(free):
            raise PageError("a page is on the free list twice")
        for p in free:
            if self._held[p]:
                raise PageError(f"page {p} is free and held")
        if len(free) + sum(self._held) != self.num_usable:
            raise PageError("a page is lost: neither free nor held")
