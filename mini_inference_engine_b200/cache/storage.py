"""Device storage behind the cache manager: pages of keys and values per layer, and per-request
state slots per layer.

Layers are grouped by need (see ``CacheLayout``); every group has its own page id space, so a
layer's tensors have as many pages as its group's pool.  A layer's pages are one tensor
``[2 (k, v), pages, kv_heads, page_size, head_dim]``: all slots of one (page, head) are contiguous,
so a kernel that works per kv head reads a page as one ``page_size x head_dim`` box.  (The
reference has one tensor ``[L, 2, NB, 16, H_kv, D]`` for all layers, inference_engine/model.py:39-53.)
Page 0 and state slot 0 are scratch: padding rows of a captured decode step read and write them.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..parts.base import KVNeed, LayerCache, StateNeed
from .manager import GroupSpec


@dataclass
class CacheLayout:
    """Which cache ids (see ``RunEntry.cache``) own which kind of storage.
    ``kv[cache id] = (group index, KVNeed)``, ``state[cache id] = StateNeed``; ``groups`` are the
    page groups in index order."""
    groups: list = field(default_factory=list)
    kv: dict = field(default_factory=dict)
    state: dict = field(default_factory=dict)

    @classmethod
    def from_needs(cls, needs: dict) -> "CacheLayout":
        """``needs[cache id]`` is what the mixer that uses it declared (None, KVNeed or StateNeed)."""
        lay = cls()
        windows = sorted({n.window for n in needs.values() if isinstance(n, KVNeed)},
                         key=lambda w: (w is not None, w or 0))
        index = {}
        for w in windows:
            index[w] = len(lay.groups)
            lay.groups.append(GroupSpec("full" if w is None else f"window{w}", w))
        for layer, n in needs.items():
            if isinstance(n, KVNeed):
                lay.kv[layer] = (index[n.window], n)
            elif isinstance(n, StateNeed):
                lay.state[layer] = n
            elif n is not None:
                raise TypeError(f"layer {layer}: cache_need() returned {type(n).__name__}")
        if not lay.groups:                      # a model without attention still gets block tables of width 0
            lay.groups.append(GroupSpec("full", None))
        return lay

    def bytes_per_page(self, group: int, page_size: int, dtype: torch.dtype) -> int:
        el = torch.empty((), dtype=dtype).element_size()
        return sum(2 * page_size * n.num_kv_heads * n.head_dim * el for g, n in self.kv.values() if g == group)

    def bytes_per_state_slot(self) -> int:
        total = 0
        for n in self.state.values():
            k = torch.empty((), dtype=n.dtype).element_size()
            for s in n.shape:
                k *= s
            total += k
        return total


class CacheStorage:
    def __init__(self, layout: CacheLayout, num_pages, page_size: int, num_state_slots: int,
                 dtype: torch.dtype, device):
        self.layout = layout
        self.page_size = page_size
        self.num_pages = list(num_pages) if isinstance(num_pages, (list, tuple)) else [num_pages] * len(layout.groups)
        self.num_state_slots = num_state_slots
        self.kv = {}
        for layer, (g, need) in layout.kv.items():
            self.kv[layer] = torch.zeros(2, self.num_pages[g], need.num_kv_heads, page_size, need.head_dim,
                                         dtype=dtype, device=device)
        self.state = {layer: torch.zeros((num_state_slots + 1,) + tuple(n.shape), dtype=n.dtype, device=device)
                      for layer, n in layout.state.items()}

    def layer_cache(self, owner: int, writes: bool = True) -> LayerCache:
        lc = LayerCache(writes=writes, page_size=self.page_size)
        if owner in self.kv:
            lc.group = self.layout.kv[owner][0]
            lc.k, lc.v = self.kv[owner][0], self.kv[owner][1]
        if owner in self.state:
            lc.state = self.state[owner]
        return lc

    def clear_state_slot(self, slot: int) -> None:
        """A request that takes a state slot starts from zero state."""
        for t in self.state.values():
            t[slot].zero_()

    def total_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in list(self.kv.values()) + list(self.state.values()))
