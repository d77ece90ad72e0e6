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

import os

import torch

from ..kernels import ops
from .base import Part, register_part

_table_cache: dict = {}
ROTATE_IN_ATTENTION = os.environ.get("MIE_B200_ROPE_IN_ATTENTION", "1") != "0"


class Rope(Part):
    def __init__(self, head_dim: int, rotary_dim: int, theta: float, max_position: int):
        if rotary_dim % 2 or rotary_dim > head_dim or rotary_dim < 0:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and at most head_dim {head_dim}")
        self.head_dim = head_dim
        self.rotary_dim = rotary_dim
        self.theta = float(theta)
        self.max_position = max_position

    def kernel_sources(self):
        return {"rope_cache"}

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

    def project_rotate_and_store(self, x, w_qkv, b_qkv, ctx, cache, num_heads, num_kv_heads):
        """The q|k|v projection followed by rotate_and_store.  Where the tensor-core product can do
        the rotation and the cache write in its epilogue (few tokens, bfloat16), that is one kernel."""
        from ..kernels import gemm_tc, linear as linear_kernels
        if (linear_kernels.uses_tcgen05(x, w_qkv) and cache.k is not None and cache.k.dtype == torch.bfloat16
                and gemm_tc.can_fuse_rope(x, w_qkv, num_heads, num_kv_heads, self.head_dim, self.rotary_dim)):
            qkv = self.rt.empty(x.shape[0], w_qkv.shape[0])
            if gemm_tc.supports(x, w_qkv, qkv):
                return gemm_tc.gemm_qkv_rope(x, w_qkv, qkv, b_qkv, ctx.positions, ctx.slots[cache.group], self.cos, self.sin,
                                             cache.k, cache.v, num_heads, num_kv_heads, self.head_dim, self.rotary_dim,
                                             cache.page_size, write_cache=cache.writes)
        qkv = self.rt.linear(x, w_qkv, b_qkv)
        self.rotate_and_store(qkv, ctx, cache, num_heads, num_kv_heads)
        return qkv

    def rotates_in_attention(self, x, w_qkv, ctx, cache) -> bool:
        """Whether the mixer should leave rotation and the cache write to its attention kernel (``tables``):
        a step of decoding rows only whose q|k|v product is the library's (above the token count that the
        tensor-core product with the rotating epilogue serves) -- one launch less a layer."""
        from ..kernels import attention as attn_kernels, linear as linear_kernels
        return (ROTATE_IN_ATTENTION and self.rotary_dim == self.head_dim and cache.k is not None and cache.writes
                and cache.k.dtype == torch.bfloat16 and not linear_kernels.uses_tcgen05(x, w_qkv)
                and attn_kernels.rotates_in_decode(x.dtype, self.head_dim, ctx))

    def tables(self):
        return self.cos, self.sin

    def rotate_and_store(self, qkv, ctx, cache, num_heads, num_kv_heads):
        ops.rope_cache_write(qkv, ctx.positions, ctx.slots[cache.group], self.cos, self.sin, cache.k, cache.v,
                             num_heads, num_kv_heads, self.head_dim, self.rotary_dim, cache.page_size,
                             write_cache=cache.writes)


class NoPosition(Rope):
    def __init__(self, head_dim: int, max_position: int):
        super().__init__(head_dim, 0, 1.0, max_position)


register_part("position", "rope", Rope)
register_part("position", "none", NoPosition)
