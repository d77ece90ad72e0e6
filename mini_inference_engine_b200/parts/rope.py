"""Rotary position encoding, rotate-half pairing (inference_engine/model.py:56-69).

Parameters: the head size, how many leading dimensions rotate (``rotary_dim``; the reference
rotates all of them), the base ``theta`` and the table length.  ``inv_freq[j] = theta^(-2j/rotary_dim)``
and the angles p * inv_freq[j] are float32; cos/sin tables are float32 too (the reference rounds
them to the model dtype, inference_engine/model.py:61).  The rotation is fused with the write of
keys and values into their cache slots, which the reference does right after it
(inference_engine/model.py:130-134).

``NoPosition`` is the same interface for a mixer without position encoding: it only stores.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part, register_part

_table_cache: dict = {}


class Rope(Part):
    def __init__(self, head_dim: int, rotary_dim: int, theta: float, max_position: int):
        if rotary_dim % 2 or rotary_dim > head_dim or rotary_dim < 0:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and at most head_dim {head_dim}")
        self.head_dim = head_dim
        self.rotary_dim = rotary_dim
        self.theta = float(theta)
        self.max_position = max_position

    def inv_freq(self) -> torch.Tensor:
        j = torch.arange(0, self.rotary_dim, 2, dtype=torch.int64).float()
        return 1.0 / (self.theta ** (j / self.rotary_dim))

    def bind(self, tensors, rt):
        self.rt = rt
        key = (str(rt.device), self.rotary_dim, self.theta, self.max_position)
        if key not in _table_cache:
            if self.rotary_dim:
                _table_cache[key] = ops.rope_tables(self.inv_freq().to(rt.device), self.max_position)
            else:
                z = torch.zeros(self.max_position, 0, dtype=torch.float32, device=rt.device)
                _table_cache[key] = (z, z)
        self.cos, self.sin = _table_cache[key]

    def rotate_and_store(self, qkv, ctx, cache, num_heads, num_kv_heads):
        ops.rope_cache_write(qkv, ctx.positions, ctx.slots[cache.group], self.cos, self.sin, cache.k, cache.v,
                             num_heads, num_kv_heads, self.head_dim, self.rotary_dim, cache.page_size,
                             write_cache=cache.writes)


class NoPosition(Rope):
    def __init__(self, head_dim: int, max_position: int):
        super().__init__(head_dim, 0, 1.0, max_position)


register_part("position", "rope", Rope)
register_part("position", "none", NoPosition)
