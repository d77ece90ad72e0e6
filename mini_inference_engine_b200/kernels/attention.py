"""Chooses the attention kernels for a step.

float32 (the true 32-bit path): the CUDA-core kernel serves every row.
bfloat16: rows with one new token go to the tensor-core decode kernel (context split across
blocks), rows with more go to a prefill kernel -- the tcgen05 one for head sizes 64 and 128, the
mma.sync one for the other multiples of 16 up to 128; head sizes beyond those kernels fall back to
the CUDA-core kernel, which takes every size up to 256.  ``set_backend("simt")`` forces the CUDA-core
kernel everywhere (used by tests to compare the two)."""
from __future__ import annotations

import torch

from . import ops

_backend = "auto"
_prefill_backend = "tcgen05"


def set_prefill_backend(name: str) -> None:
    global _prefill_backend
    if name not in ("tcgen05", "mma"):
        raise ValueError(name)
    _prefill_backend = name


def set_backend(name: str) -> None:
    global _backend
    if name not in ("auto", "simt"):
        raise ValueError(name)
    _backend = name


def _row_kinds(ctx) -> tuple:
    """(rows of one token, rows of more, tokens of those) of the step, or None where the host does not know the rows'
    lengths (a captured step).  Counted once a step, not once a layer: a step may hold hundreds of rows."""
    kinds = ctx.host.get("_row_kinds", False)
    if kinds is False:
        q_lens = ctx.host.get("q_len")
        kinds = None
        if q_lens is not None:
            long = [n for n in q_lens if n > 1]
            kinds = (len(q_lens) - len(long), len(long), sum(long))
        ctx.host["_row_kinds"] = kinds
    return kinds


def decode_only(ctx) -> bool:
    """Whether every row of the step has exactly one new token (known on the host)."""
    kinds = _row_kinds(ctx)
    return kinds is not None and kinds[1] == 0 and kinds[0] > 0


def rotates_in_decode(dtype, head_dim: int, ctx) -> bool:
    """Whether ``attention(..., rope=...)`` can rotate q and the new key itself and write the cache: a step of
    decoding rows only, on the tensor-core decode kernel, with a head size it rotates."""
    return (_backend == "auto" and dtype == torch.bfloat16 and head_dim <= 128 and head_dim % 32 == 0
            and decode_only(ctx))


def attention(qkv, ctx, cache, out, num_heads, num_kv_heads, head_dim, scale, window, rope=None):
    """``rope`` = (cos, sin): ``qkv`` is unrotated and the cache rows of the new tokens are unwritten; only
    where ``rotates_in_decode`` holds."""
    q_stride = (num_heads + 2 * num_kv_heads) * head_dim
    args = (qkv, q_stride, cache.k, cache.v, ctx.block_tables[cache.group], ctx.row_q_start, ctx.row_q_len,
            ctx.row_ctx_len)
    fast = _backend == "auto" and qkv.dtype == torch.bfloat16 and head_dim <= 128
    if rope is not None:
        if not rotates_in_decode(qkv.dtype, head_dim, ctx):
            raise ValueError("rotation inside attention serves steps of decoding rows only (bfloat16, head sizes "
                             "in steps of 32 up to 128)")
        return ops.decode_attention(*args, out, num_heads, num_kv_heads, head_dim, cache.page_size, scale, window,
                                    max_ctx=ctx.max_ctx_len, rope=rope)
    if not fast:
        return ops.paged_attention(*args, ctx.num_tokens, out, num_heads, num_kv_heads, head_dim, cache.page_size,
                                   scale, window)
    kinds = _row_kinds(ctx)
    has_decode = kinds is None or kinds[0] > 0
    has_prefill = kinds is None or kinds[1] > 0
    min_q_len = 2
    if kinds is None and ctx.host.get("few_single_rows"):
        # row lengths unknown here (a captured step), but rows of one token are the exception among them: the
        # kernel for portions takes those too, and the launch of the decode kernel is saved
        has_decode, min_q_len = False, 1
    if has_decode:
        ops.decode_attention(*args, out, num_heads, num_kv_heads, head_dim, cache.page_size, scale, window,
                             max_ctx=ctx.max_ctx_len)
    if has_prefill:
        # tcgen05 (S and O in tensor memory) for the head sizes it is written for, mma.sync otherwise
        tc = head_dim in (64, 128) and cache.page_size >= 8 and q_stride % 8 == 0 and _prefill_backend == "tcgen05"
        fn = ops.prefill_attention_tc if tc else ops.prefill_attention
        # the rows that are portions, and their tokens: the launch is laid out for those, not for every decoding row
        work = None if kinds is None else (kinds[1], kinds[2])
        fn(*args, ctx.num_tokens, out, num_heads, num_kv_heads, head_dim, cache.page_size, scale, window,
           min_q_len=min_q_len, work=work)
    return out
