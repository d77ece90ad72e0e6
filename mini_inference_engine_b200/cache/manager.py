"""The cache manager: which pages and which state slot each live request holds.

Layers are put into *groups* by what they need of the past: ``full`` groups keep every key
and value, ``window`` groups keep only the last ``window`` positions.  Every group has pages
of its own (its own pool and its own device tensors), because a page of a window group can go
back to the pool as soon as the window has passed it while the same positions are still held
in a full group.  A request has one block table per group: logical page i -> physical page id,
``RELEASED`` (0, the scratch page) once the window has passed.  Beside the pages there are
slots for per-request state of fixed size (what a recurrent mixer would carry); Llama's
attention has none, so the slot tensors are empty, but the slot ids are handed out, passed to
the step function and given back all the same.

The reference has one group, no windows and no state (inference_engine/block_manager.py:14-44,
inference_engine/model.py:39-53); the rules it has are kept: pages are reserved for the next n
tokens before a step (``reserve``), admissions must leave ``watermark`` pages free, growth of a
running request ignores the watermark, and everything is given back at once when a request
ends or is preempted (inference_engine/scheduler.py:38-45,104-107).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .pages import PageError, PagePool

RELEASED = 0   # block-table entry of a page the window has passed: the scratch page


@dataclass(frozen=True)
class GroupSpec:
    """A group of layers with the same need: ``window`` None keeps all positions."""
    name: str
    window: int | None = None


@dataclass
class RequestCache:
    """What one request holds.  ``tables[g][i]`` is the physical page of logical page i in
    group g; ``first_live[g]`` is the first logical page not yet released."""
    tables: list = field(default_factory=list)
    first_live: list = field(default_factory=list)
    state_slot: int = 0
    num_computed: int = 0
    version: int = 0                  # counts the changes of ``tables`` (the manager bumps it)
    _arrays: tuple = field(default=(-1, None), repr=False, compare=False)

    def table_arrays(self) -> list:
        """``tables`` as int32 arrays, made again only after a change: a running request's table
        changes once a page, the batch builder wants it every step.  Read-only by agreement."""
        if self._arrays[0] != self.version:
            self._arrays = (self.version, [np.array(t, dtype=np.int32) for t in self.tables])
        return self._arrays[1]


class CacheManager:
    def __init__(self, groups: list[GroupSpec], num_pages: int | list[int], block_size: int,
                 num_state_slots: int = 0):
        if not groups:
            raise ValueError("at least one cache group is needed")
        self.groups = list(groups)
        self.block_size = block_size
        counts = num_pages if isinstance(num_pages, (list, tuple)) else [num_pages] * len(groups)
        self.pools = [PagePool(n) for n in counts]
        self._windowed = any(g.window is not None for g in self.groups)
        # slot 0 is the scratch slot of padding rows, like page 0
        self.state_pool = PagePool(num_state_slots + 1) if num_state_slots > 0 else None

    # ------------------------------------------------------------------ sizes
    def _first_needed_page(self, g: int, num_computed: int) -> int:
        w = self.groups[g].window
        if w is None:
            return 0
        # the next query is at position num_computed and reads keys > num_computed - w
        return max(0, num_computed - w + 1) // self.block_size

    def pages_needed(self, rc: RequestCache, n_new: int) -> list[int]:
        """Pages each group still lacks to hold positions up to num_computed + n_new."""
        total = rc.num_computed + n_new
        last = -(-total // self.block_size)
        self._ensure_tables(rc)
        return [max(0, last - len(rc.tables[g])) for g in range(len(self.groups))]

    def max_pages_for(self, num_tokens: int) -> list[int]:
        """The most pages a request of ``num_tokens`` positions holds at any time, per group,
        when it is fed in one portion (the worst case)."""
        return [-(-num_tokens // self.block_size) for _ in self.groups]

    def num_free(self, g: int = 0) -> int:
        return self.pools[g].num_free

    def _ensure_tables(self, rc: RequestCache) -> None:
        if not rc.tables:
            rc.tables = [[] for _ in self.groups]
            rc.version += 1
            rc.first_live = [0 for _ in self.groups]

    # ------------------------------------------------------------------ reserve / advance / free
    def can_reserve(self, rc: RequestCache, n_new: int, watermark: int = 0) -> bool:
        need = self.pages_needed(rc, n_new)
        return all(self.pools[g].can_take(need[g], watermark) for g in range(len(self.groups)))

    def reserve(self, rc: RequestCache, n_new: int, watermark: int = 0) -> bool:
        """Makes sure the request has pages for its next ``n_new`` tokens in every group; takes
        nothing when any group cannot give what is needed."""
        last = -(-(rc.num_computed + n_new) // self.block_size)
        if rc.tables and all(len(t) >= last for t in rc.tables):
            return True                       # the common case of a decode step: the last page has room
        need = self.pages_needed(rc, n_new)
        if not all(self.pools[g].can_take(need[g], watermark) for g in range(len(self.groups))):
            return False
        for g, n in enumerate(need):
            if n:
                rc.tables[g].extend(self.pools[g].take(n))
                rc.version += 1
        return True

    def take_state_slot(self, rc: RequestCache) -> bool:
        if self.state_pool is None or rc.state_slot:
            return True
        if not self.state_pool.can_take(1):
            return False
        rc.state_slot = self.state_pool.take(1)[0]
        return True

    def advance(self, rc: RequestCache, n: int) -> list[list[int]]:
        """The step wrote ``n`` more positions.  Gives back the pages that every window has
        passed; returns them per group (for tests)."""
        rc.num_computed += n
        released = [[] for _ in self.groups]
        if not self._windowed:
            return released
        for g in range(len(self.groups)):
            first = min(self._first_needed_page(g, rc.num_computed), len(rc.tables[g]))
            for i in range(rc.first_live[g], first):
                p = rc.tables[g][i]
                if p != RELEASED:
                    released[g].append(p)
                    rc.tables[g][i] = RELEASED
            if released[g]:
                self.pools[g].give_back(released[g])
                rc.version += 1
            rc.first_live[g] = max(rc.first_live[g], first)
        return released

    def free(self, rc: RequestCache) -> None:
        """Everything the request holds goes back (end of the request, or preemption)."""
        self._ensure_tables(rc)
        for g in range(len(self.groups)):
            self.pools[g].give_back([p for p in rc.tables[g] if p != RELEASED])
        rc.tables = [[] for _ in self.groups]
        rc.version += 1
        rc.first_live = [0 for _ in self.groups]
        rc.num_computed = 0
        if self.state_pool is not None and rc.state_slot:
            self.state_pool.give_back([rc.state_slot])
        rc.state_slot = 0

    def check(self) -> None:
        for p in self.pools:
            p.check()
        if self.state_pool is not None:
            self.state_pool.check()


__all__ = ["CacheManager", "GroupSpec", "RequestCache", "RELEASED", "PageError"]
