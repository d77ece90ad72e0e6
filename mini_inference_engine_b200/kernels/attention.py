"""Chooses the attention kernel for a step.  The CUDA-core kernel serves every case in both
types; tensor-core kernels for bfloat16 take over the cases they are written for."""
from __future__ import annotations

from . import ops

_backend = "auto"


def set_backend(name: str) -> None:
    global _backend
    if name not in ("auto", "simt"):
        raise ValueError(name)
    _backend = name


def attention(qkv, ctx, cache, out, num_heads, num_kv_heads, head_dim, scale, window):
    q_stride = (num_heads + 2 * num_kv_heads) * head_dim
    return ops.paged_attention(qkv, q_stride, cache.k, cache.v, ctx.block_tables[cache.group], ctx.row_q_start,
                               ctx.row_q_len, ctx.row_ctx_len, ctx.num_tokens, out, num_heads, num_kv_heads,
                               head_dim, cache.page_size, scale, window)
