"""Python faces of the CUDA kernels: each function checks shapes and types, then calls the
``extern "C"`` launcher of its library on torch's current stream.  Tensors are passed as raw
device pointers; nothing here computes on the host or through a library kernel, and there is no
other path: a tensor that is not on a CUDA device is refused.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import build
from .device import num_sms

F32, BF16 = 0, 1
_TAGS = {torch.float32: F32, torch.bfloat16: BF16}

_CUDA_ERRORS = {-1: "a size or option the kernel does not take", -2: "beyond the kernel's stated maximum"}


class KernelError(RuntimeError):
    pass


def tag(t: torch.Tensor) -> int:
    try:
        return _TAGS[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported element type {t.dtype}; kernels take float32 and bfloat16") from None


def _ptr(t):
    if t is None:
        return ctypes.c_void_p(0)
    if not t.is_cuda:
        raise KernelError("kernels of this package run on CUDA tensors only; got a tensor on " + str(t.device))
    return ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


before_launch: list = []     # callables run before any launch of this package (a pending chain of products goes first)


def _stream():
    """The current CUDA stream's handle.  Asked on every launch (a graph capture switches streams)."""
    for hook in before_launch:
        hook()
    return raw_stream()


def raw_stream():
    if _raw_stream is not None:                      # the direct query; a tenth of the cost of the Stream object
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


launches = 0        # kernels of this package launched so far (captured launches count once, at capture)


def _check(code: int, what: str) -> None:
    global launches
    if code == 0:
        launches += 1
        return
    if code < 0:
        raise KernelError(f"{what}: refused, {_CUDA_ERRORS.get(code, code)}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


# --------------------------------------------------------------------------- range report
# Four int32 in pinned host memory that the kernels write directly (code, kernel, index, value): see
# csrc/range_check.cuh.  Every library that checks ranges is told the address when it is loaded.
_RANGE_CODES = {1: "token id outside the vocabulary (or the fed-back tokens)", 2: "position outside the position table "
                "(or more positions than the block table covers)", 3: "cache slot outside the cache",
                4: "block-table entry outside the page pool", 5: "row index outside the batch"}
_RANGE_KERNELS = {1: "embedding", 2: "rope_cache", 3: "norm", 4: "attention_simt", 5: "attention_decode",
                  6: "attention_prefill", 7: "attention_prefill_tc", 8: "gemm_tcgen05 (q|k|v with rotation)"}
_range_report: torch.Tensor | None = None
_range_told: set = set()


def range_report() -> torch.Tensor:
    global _range_report
    if _range_report is None:
        with torch.inference_mode(False):        # made inside a step, it would refuse to be cleared outside one
            _range_report = torch.zeros(4, dtype=torch.int32, pin_memory=True)
    return _range_report


def load(name: str):
    """The library of ``csrc/<name>.cu``, told where the range report lives if it checks ranges."""
    lib = build.load(name)
    if name not in _range_told:
        _range_told.add(name)
        if hasattr(lib, "mie_set_range_report"):
            lib.mie_set_range_report(ctypes.c_void_p(range_report().data_ptr()))
    return lib


def check_range_errors() -> None:
    """Raises if a kernel met an integer out of range since the last call (after a synchronise): the
    kernel skipped that access, so the step's result is not valid."""
    if _range_report is None:
        return
    code, kernel, index, value = _range_report.tolist()
    if code:
        _range_report.numpy()[:] = 0
        raise KernelError(f"{_RANGE_KERNELS.get(kernel, kernel)}: {_RANGE_CODES.get(code, code)}: "
                          f"value {value} at index {index}; the access was skipped and the step's output is not valid")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _i32(t, name):
    _need(t.dtype == torch.int32 and t.is_contiguous(), f"{name} must be a contiguous int32 tensor")


# --------------------------------------------------------------------------- embedding

def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, feedback: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = table[ids[t]] as float32 (the residual stream).  An id -(k+1) is replaced on the device
    by ``feedback[k]`` (a token the previous step sampled and the host has not read yet)."""
    if feedback is not None:
        _i32(feedback, "feedback")
    _i32(ids, "ids")
    V, h = table.shape
    _need(out.dtype == torch.float32 and out.shape == (ids.numel(), h) and out.is_contiguous(),
          "embedding output must be contiguous float32 [tokens, hidden]")
    _need(table.is_contiguous(), "embedding table must be contiguous")
    lib = load("embedding")
    _check(lib.mie_embedding(_ptr(table), tag(table), _ptr(ids), _ptr(feedback), _ptr(out), ids.numel(), h, V,
                             feedback.numel() if feedback is not None else 0, _stream()),
           "embedding")
    return out


# --------------------------------------------------------------------------- norm

def add_rmsnorm(delta, res: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: torch.Tensor | None = None) -> torch.Tensor:
    """res += delta (in place, float32); out = rmsnorm(res) * weight.  With ``rows`` the inputs are
    gathered (output row b from input row rows[b]) and ``res`` is not written."""
    n = res.shape[-1]
    _need(res.dtype == torch.float32 and res.is_contiguous(), "the residual stream must be contiguous float32")
    _need(out.is_contiguous() and out.shape[-1] == n, "norm output must be contiguous [rows, n]")
    _need(weight.numel() == n and weight.is_contiguous(), f"norm weight must have {n} entries")
    if delta is not None:
        _need(delta.dtype == out.dtype and delta.shape == res.shape and delta.is_contiguous(),
              "delta must match the residual's shape and the output's type")
    num_rows = out.shape[0]
    if rows is not None:
        _i32(rows, "rows")
        _need(rows.numel() == num_rows, "one gathered row per output row")
    else:
        _need(res.shape[0] == num_rows, "output rows must match residual rows")
    lib = load("norm")
    _check(lib.mie_add_rmsnorm(_ptr(delta), _ptr(res), _ptr(weight), tag(weight), _ptr(out), tag(out),
                               _ptr(rows), num_rows, n, ctypes.c_float(eps), res.shape[0], _stream()), "add_rmsnorm")
    return out


# --------------------------------------------------------------------------- rope + cache write

def rope_tables(inv_freq: torch.Tensor, max_pos: int):
    """cos, sin [max_pos, rotary_dim/2] float32 of p * inv_freq[j]."""
    _need(inv_freq.dtype == torch.float32 and inv_freq.is_contiguous(), "inv_freq must be float32")
    half = inv_freq.numel()
    cos = torch.empty(max_pos, half, dtype=torch.float32, device=inv_freq.device)
    sin = torch.empty_like(cos)
    lib = build.load("rope_cache")
    _check(lib.mie_rope_table(_ptr(inv_freq), _ptr(cos), _ptr(sin), max_pos, half, _stream()), "rope_table")
    return cos, sin


def rope_cache_write(qkv: torch.Tensor, positions, slots, cos, sin, k_cache, v_cache, num_heads: int,
                     num_kv_heads: int, head_dim: int, rotary_dim: int, page_size: int,
                     write_cache: bool = True) -> None:
    """Rotates q in place inside ``qkv`` [T, (H + 2 H_kv) D] and writes rotated k and v into their
    cache slots (pages laid out [page, kv_head, slot, D])."""
    T = qkv.shape[0]
    _need(qkv.is_contiguous() and qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim,
          "qkv must be contiguous [tokens, (H + 2 H_kv) * D]")
    _i32(positions, "positions")
    _i32(slots, "slots")
    _need(k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype, "cache type must match qkv")
    _need(cos.shape[1] * 2 == rotary_dim, "rotation table does not match rotary_dim")
    lib = load("rope_cache")
    _check(lib.mie_rope_cache_write(_ptr(qkv), tag(qkv), _ptr(positions), _ptr(slots), _ptr(cos), _ptr(sin),
                                    _ptr(k_cache), _ptr(v_cache), T, num_heads, num_kv_heads, head_dim,
                                    rotary_dim, page_size, cos.shape[0], int(write_cache),
                                    ctypes.c_longlong(k_cache.shape[0]), _stream()),
           "rope_cache_write")


# --------------------------------------------------------------------------- attention

def paged_attention(q: torch.Tensor, q_stride: int, k_cache, v_cache, block_tables, row_q_start, row_q_len,
                    row_ctx_len, num_tokens: int, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                    head_dim: int, page_size: int, scale: float, window: int | None = None,
                    min_q_len: int = 1) -> torch.Tensor:
    """Causal attention of every new token over its request's pages (CUDA-core kernel, float32 or
    bfloat16).  ``q`` holds [H, D] at the start of each token row of ``q_stride`` elements.  Rows
    with fewer than ``min_q_len`` new tokens are left alone."""
    _need(head_dim % 16 == 0 and 16 <= head_dim <= 256,
          f"head_dim {head_dim}: this kernel takes multiples of 16 from 16 to 256")
    _need(num_heads % num_kv_heads == 0, "query heads must be a multiple of kv heads")
    for t, n in ((block_tables, "block_tables"), (row_q_start, "row_q_start"), (row_q_len, "row_q_len"),
                 (row_ctx_len, "row_ctx_len")):
        _i32(t, n)
    _need(out.dtype == q.dtype == k_cache.dtype == v_cache.dtype, "q, caches and out must share a type")
    _need(out.is_contiguous(), "attention output must be contiguous")
    rows = row_q_len.numel()
    lib = load("attention_simt")
    _check(lib.mie_paged_attention(_ptr(q), ctypes.c_int64(q_stride), _ptr(k_cache), _ptr(v_cache),
                                   _ptr(block_tables), block_tables.shape[1], _ptr(row_q_start), _ptr(row_q_len),
                                   _ptr(row_ctx_len), rows, num_tokens, _ptr(out), tag(q), num_heads,
                                   num_kv_heads, head_dim, page_size, ctypes.c_float(scale),
                                   int(window or 0), int(min_q_len), ctypes.c_longlong(k_cache.shape[0]), _stream()),
           "paged_attention")
    return out


def prefill_attention(q: torch.Tensor, q_stride: int, k_cache, v_cache, block_tables, row_q_start, row_q_len,
                      row_ctx_len, num_tokens: int, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                      head_dim: int, page_size: int, scale: float, window: int | None = None,
                      min_q_len: int = 2, work=None) -> torch.Tensor:
    """Causal attention of prompt portions over their request's pages (bfloat16, tensor cores).
    Rows with fewer than ``min_q_len`` new tokens are left alone.  ``work`` = (rows, tokens): how many rows have
    ``min_q_len`` tokens or more and their tokens in sum, where the caller knows -- the launch then has blocks for the
    tiles those rows can have, not for every row of the step."""
    _need(q.dtype == torch.bfloat16 == k_cache.dtype == v_cache.dtype == out.dtype, "prefill attention is bfloat16")
    _need(head_dim % 16 == 0 and 16 <= head_dim <= 128,
          f"head_dim {head_dim}: the prefill kernel takes multiples of 16 from 16 to 128")
    _need(num_heads % num_kv_heads == 0, "query heads must be a multiple of kv heads")
    for t, n in ((block_tables, "block_tables"), (row_q_start, "row_q_start"), (row_q_len, "row_q_len"),
                 (row_ctx_len, "row_ctx_len")):
        _i32(t, n)
    _need(out.is_contiguous(), "attention output must be contiguous")
    lib = load("attention_prefill")
    _check(lib.mie_prefill_attention(_ptr(q), ctypes.c_int64(q_stride), _ptr(k_cache), _ptr(v_cache),
                                     _ptr(block_tables), block_tables.shape[1], _ptr(row_q_start), _ptr(row_q_len),
                                     _ptr(row_ctx_len), row_q_len.numel(), num_tokens, _ptr(out), num_heads,
                                     num_kv_heads, head_dim, page_size, ctypes.c_float(scale), int(window or 0),
                                     int(min_q_len), ctypes.c_longlong(k_cache.shape[0]), *_work_args(work), _stream()),
           "prefill_attention")
    return out


def prefill_attention_tc(q: torch.Tensor, q_stride: int, k_cache, v_cache, block_tables, row_q_start, row_q_len,
                         row_ctx_len, num_tokens: int, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                         head_dim: int, page_size: int, scale: float, window: int | None = None,
                         min_q_len: int = 2, work=None) -> torch.Tensor:
    """Causal attention of prompt portions on tcgen05 (S and O in tensor memory, operands by TMA);
    head_dim 64 or 128.  ``work``: as for ``prefill_attention``."""
    _need(q.dtype == torch.bfloat16 == k_cache.dtype == v_cache.dtype == out.dtype, "prefill attention is bfloat16")
    _need(head_dim in (64, 128), f"head_dim {head_dim}: the tcgen05 prefill kernel takes 64 and 128")
    _need(q_stride % 8 == 0 and page_size >= 8, "the tcgen05 prefill kernel needs q rows and pages of whole 16-byte pieces")
    _need(num_heads % num_kv_heads == 0, "query heads must be a multiple of kv heads")
    for t, n in ((block_tables, "block_tables"), (row_q_start, "row_q_start"), (row_q_len, "row_q_len"),
                 (row_ctx_len, "row_ctx_len")):
        _i32(t, n)
    _need(out.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous(), "contiguous caches and output")
    lib = load("attention_prefill_tc")
    _check(lib.mie_prefill_attention_tc(_ptr(q), ctypes.c_int64(q_stride), _ptr(k_cache), _ptr(v_cache),
                                        ctypes.c_int64(k_cache.shape[0]), _ptr(block_tables), block_tables.shape[1],
                                        _ptr(row_q_start), _ptr(row_q_len), _ptr(row_ctx_len), row_q_len.numel(),
                                        num_tokens, _ptr(out), num_heads, num_kv_heads, head_dim, page_size,
                                        ctypes.c_float(scale), int(window or 0), int(min_q_len), *_work_args(work), _stream()),
           "prefill_attention_tc")
    return out


def _work_args(work):
    rows, tokens = work if work is not None else (0, 0)
    return int(rows), int(tokens)


def set_prefill_pairs(mode: int = -1) -> None:
    """Which tcgen05 prefill kernel serves head_dim 64: -1 chooses by the size of the launch (the default), 0 always
    one query tile a block, 1 always two query tiles side by side (csrc/attention_prefill_tc.cu)."""
    load("attention_prefill_tc").mie_prefill_attention_tc_pairs(int(mode))


def check_tc_errors() -> None:
    """Raises if a block of a tensor-core kernel gave up a bounded wait (call after a synchronise)."""
    for name, fn in (("attention_prefill_tc", "mie_prefill_attention_tc"), ("attention_decode", "mie_decode_attention")):
        lib = build._libs.get(name)
        if lib is not None and getattr(lib, fn + "_error")():
            getattr(lib, fn + "_clear_error")()
            raise KernelError(f"a block of {name} gave up waiting on a barrier; its output is not valid")


_workspaces: dict = {}
_outgrown: list = []          # scratch tensors that a larger one replaced; see _workspace


def _workspace(device, name: str, numel: int, dtype) -> torch.Tensor:
    """A persistent, zero-initialised scratch tensor per (device, name), grown on demand.  Kernels
    that use it leave it as they need to find it, so it is cleared only when it is (re)made.  A captured
    graph keeps the ADDRESS of the tensor it was captured with, so a tensor that has been outgrown is kept
    alive, never handed back to the allocator: graphs captured with it go on using it (each scratch tensor
    is self-contained, and the launches of one stream use them one after the other).  Sizes at least
    double, which bounds what is kept."""
    key = (str(device), name)
    t = _workspaces.get(key)
    if t is None or t.numel() < numel:
        if t is not None:
            _outgrown.append(t)
            numel = max(numel, 2 * t.numel())
        t = torch.zeros(max(numel, 1024), dtype=dtype, device=device)
        _workspaces[key] = t
    return t


def decode_splits(rows: int, kv_units: int, max_ctx: int, head_dim: int = 64) -> int:
    """How many parts to cut the context into (a cluster of 2, 4 or 8 blocks; the reference keeps 256 keys a
    part, inference_engine/kernels/decode_attention.py:117-125).

    Heads of up to 64: as many parts as still leave every block a place beside the others -- four blocks on an SM
    with page copies by TMA and two stages (``decode_uses_tma``, ``decode_stages``) -- and two 64-key tiles a part.
    Measured on B200 (32 q / 4 kv heads of 64, device time in a graph, context bound 960; the plan before ->
    this one): 512 keys, 20 / 32 rows 7.1 -> 6.4 / 8.2 -> 7.0 us (4 parts), 40 / 64 / 72 rows 10.5 -> 8.7 / 11.6 -> 9.2 /
    12.0 -> 9.4 us (2 parts), 80 / 96 rows 20.4 -> 11.3 / 20.6 -> 11.6 us (whole, by TMA, four stages); 960 keys, 16
    rows 8.4 -> 7.3 us (8 parts), 24 rows 11.8 -> 9.0, 64 rows 19.7 -> 14.2, 96 rows 36.4 -> 19.6 us.  One block
    more than the places (592) and the launch takes half as long again: 72 rows in two parts 9.4 us, 80 rows 16.3.
    Wider heads (two blocks on an SM): parts while the batch alone leaves SMs idle."""
    blocks = max(1, rows * kv_units)
    splits = 1
    if head_dim <= 64:
        most = -(-(-(-max(1, max_ctx) // 64)) // 2)            # two tiles a part at least
        while splits < 8 and blocks * splits * 2 <= decode_blocks_per_sm(head_dim) * num_sms() and splits * 2 <= most:
            splits *= 2
        return splits
    while splits < 8 and blocks * splits * 2 <= 2 * num_sms() and splits * 64 < max_ctx:
        splits *= 2
    return splits


LONG_PART_TILES = 8          # a part of a long context is at least this many 64-key tiles (512 keys)


def decode_blocks_per_sm(head_dim: int) -> int:
    """Blocks of the decode kernel that share an SM with page copies by TMA and three stages: a stage is 16 KB of
    keys and values per 64 columns of the head, beside 6 KB of static shared memory."""
    return 4 if head_dim <= 64 else 2


def decode_plan(rows: int, kv_units: int, max_ctx: int, tma_ok: bool, head_dim: int = 64) -> tuple[int, str, int]:
    """(splits, merge, min_part_tiles) for a decode launch whose contexts reach up to ``max_ctx``.

    Short contexts and few rows: the cluster merge of ``decode_splits`` (one launch, no global round trip).
    Long contexts (two parts of LONG_PART_TILES tiles or more) with 64 or more (row, kv head) units: a block
    walks its keys at about 16 ns a key whatever else runs (three or four 16 KB tiles in flight), so the
    bytes per second follow the number of blocks that run beside one another -- four per SM (two with heads
    of 128) with page copies by TMA, three stages and no receive slots of a cluster.  The context is then cut into as many
    parts as fill those places, merged through scratch memory, and a row shorter than the launch was laid
    out for is cut into fewer parts by the kernel (``min_part_tiles``).  Measured on B200, 32 q / 4 kv
    heads of 64, device time in a graph, cluster plan -> this plan: 64 rows x 8,192 keys 149 -> 90 us
    (5.96 TB/s), 32 x 8,192 72 -> 48 us, 16 x 8,192 38 -> 31 us, 64 x 2,048 36.8 -> 31.0 us, 32 x 2,048
    20.5 -> 17.8 us; 8 rows stay with the cluster of 8 (20.9 us at 8,192 keys against 24.2 us).  With 8 kv
    heads of 128 (32 rows x 2,048 keys) the whole context per block is the fastest plan (46.3 us; two parts
    62.7 us): 256 blocks already fill the two places an SM has."""
    units = max(1, rows * kv_units)
    clustered = decode_splits(rows, kv_units, max_ctx, head_dim)
    tiles = -(-max(1, max_ctx) // 64)
    if tma_ok and units >= 64 and tiles >= 2 * LONG_PART_TILES:
        parts = min(decode_blocks_per_sm(head_dim) * num_sms() // units, tiles // LONG_PART_TILES, 8 if head_dim <= 64 else 16)
        # Only where scratch allows MORE parts than a cluster (which takes 2, 4 or 8): with as many parts the cluster
        # is the faster merge (heads of 64, page copies by TMA, two stages; rows x keys, scratch -> cluster:
        # 64 x 2,048 31.5 -> 25.6 us, 64 x 3,400 45.5 -> 39.6, 32 x 2,048 18.2 -> 14.6, 16 x 2,048 17.6 -> 10.0 us);
        # three parts through scratch against two of a cluster win from about 3,400 keys on (48 x 7,000: 63.9
        # against 71.9 us; 48 x 2,048: 27.0 against 24.0 us)
        if parts >= 2 and parts > clustered:
            return parts, "scratch", LONG_PART_TILES
    return clustered, "cluster", 0


def decode_stages(blocks: int, max_ctx: int, splits: int, tma: bool = False, head_dim: int = 64, clustered: bool = True) -> int:
    """Tiles of 64 keys in flight per block.  Shared memory that attention does not take stays free
    for the prologue of the kernel after it (the output projection fills its ring with weights while
    attention still runs): measured on B200 in the whole decode step at batch 8, 512 keys, three
    stages 1.069 ms, four 1.087 ms, two 1.135 ms (two stages are slower by themselves).  Parts of
    more than four tiles want the deepest ring (batch 64, 512 keys: 12.7 us with four stages, 15.5 us
    with three; 2048 keys: 40 us with four, 60 us with two); more blocks than fit beside one another
    at four stages want two, which puts twice as many on an SM (batch 256, 512 keys: 34 us against
    46 us).  Heads of 128 with TMA copies: three stages (two blocks on an SM) up to six blocks per SM in the
    launch, two stages (three on an SM) beyond (32 kv heads of 128, 512 keys: 64 rows 87.9 against 98.0 us, 32 rows
    51.4 against 53.9 us; 8 kv heads, 64 rows 32.3 against 27.7 us)."""
    tiles = -(-(-(-max(1, max_ctx) // splits)) // 64)
    if head_dim > 64 and tma:
        return 2 if blocks > 6 * num_sms() else 3
    if tma and splits > 1 and clustered:
        return 2                          # the parts of a cluster by TMA: four blocks on an SM (see decode_splits)
    if tma and blocks <= 3 * num_sms():
        return 4                          # whole contexts by TMA, up to three blocks an SM (80 rows x 512 keys: 11.3 us; 128 rows want three stages: 13.0 against 21.0 us)
    if blocks > 3 * num_sms():
        return 3 if tma else 2            # TMA tiles are unpadded: three stages still put four blocks on an SM (256 x 512: 29.2 us, two stages 30.7)
    return 3 if tiles <= 4 else 4


def decode_uses_tma(blocks: int, head_dim: int = 64) -> bool:
    """Whether the decode kernel fetches keys and values a page per TMA copy instead of 16 bytes per
    cp.async.  Measured on B200 (32 q / 4 kv heads of 64): it pays where there are more blocks than
    fit beside one another at three or four padded stages of 16-byte copies, from two blocks per SM on (128 requests
    x 512 keys: 14.9 us against 20.6 us; 256 x 512: 29.2 against 34.4 us; 80 x 512, whole contexts: 11.3 against
    20.4 us; 16 x 960 in 8 parts: 7.3 against 12.0 us) and costs a little where each block walks a long part alone (64 x 2048: 42.9 against
    40.0 us; 8 x 512: 7.5 against 7.1 us) -- the copies were never the bound there, the softmax
    bookkeeping per 16 keys is.  Cache slots beyond a request's context are copied along with their
    page and must hold finite values (the cache storage starts as zeros).  Heads of 128: always -- a stage of
    cp.async copies is 34 KB there and the 16-byte copies are four times as many (8 rows x 512 keys, 8 kv heads:
    7.3 against 14.2 us; 1,024 keys 9.8 against 20.4 us; 32 kv heads, 1 row x 512 keys: 6.2 against 14.4 us)."""
    return head_dim > 64 or blocks > 2 * num_sms()


def decode_attention(q: torch.Tensor, q_stride: int, k_cache, v_cache, block_tables, row_q_start, row_q_len,
                     row_ctx_len, out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                     page_size: int, scale: float, window: int | None = None, max_ctx: int = 0,
                     splits: int | None = None, merge: str | None = None, stages: int | None = None,
                     tma: bool | None = None, min_part_tiles: int = 0, rope=None) -> torch.Tensor:
    """Attention of rows with exactly one new token (bfloat16, tensor cores, context split across
    blocks and merged in the same launch).  Rows with more new tokens are skipped.  ``merge`` =
    "cluster": 1, 2, 4 or 8 splits merged through distributed shared memory; "scratch": any number of
    splits merged through scratch memory in global memory, a row cut into at most (its tiles /
    ``min_part_tiles``) of them.  With neither ``splits`` nor ``merge`` given, ``decode_plan`` chooses.

    ``rope`` = (cos, sin), float32 [positions, head_dim / 2]: ``q`` holds the UNROTATED q|k|v activation of
    every row (keys ``num_heads`` heads in, values behind them), and the kernel rotates q and the new key by the
    row's position (context length - 1, the whole head as rotary width), uses them, and writes the new key and
    value into the cache -- the separate rotate-and-store launch is not needed then."""
    _need(q.dtype == torch.bfloat16 == k_cache.dtype == v_cache.dtype == out.dtype, "decode attention is bfloat16")
    _need(head_dim % 16 == 0 and 16 <= head_dim <= 128,
          f"head_dim {head_dim}: the decode kernel takes multiples of 16 from 16 to 128")
    _need(num_heads % num_kv_heads == 0, "query heads must be a multiple of kv heads")
    for t, n in ((block_tables, "block_tables"), (row_q_start, "row_q_start"), (row_q_len, "row_q_len"),
                 (row_ctx_len, "row_ctx_len")):
        _i32(t, n)
    rows = row_q_len.numel()
    cos = sin = None
    if rope is not None:
        cos, sin = rope
        _need(head_dim % 32 == 0, f"head_dim {head_dim}: rotation inside the decode kernel takes multiples of 32")
        _need(cos.dtype == torch.float32 == sin.dtype and cos.is_contiguous() and sin.is_contiguous()
              and cos.shape == sin.shape and cos.dim() == 2 and cos.shape[1] == head_dim // 2,
              "rope tables must be contiguous float32 [positions, head_dim / 2]")
        _need(q_stride >= (num_heads + 2 * num_kv_heads) * head_dim and q_stride % 8 == 0,
              "rotation inside the decode kernel reads q|k|v rows (16-byte aligned)")
    chunks = -(-(num_heads // num_kv_heads) // 16)
    tma_ok = head_dim in (64, 128) and page_size >= 8
    if splits is None and merge is None:
        splits, merge, min_part_tiles = decode_plan(rows, num_kv_heads * chunks, max_ctx or 1, tma_ok and tma is not False,
                                                    head_dim)
        if merge == "scratch" and tma is None:
            tma = True
    elif splits is None:
        splits = decode_splits(rows, num_kv_heads * chunks, max_ctx or 1, head_dim)
    merge = merge or "cluster"
    if tma is None:
        tma = decode_uses_tma(rows * num_kv_heads * chunks * splits, head_dim)
    tma = bool(tma) and tma_ok
    if stages is None:
        stages = decode_stages(rows * num_kv_heads * chunks * splits, max_ctx or 4096, splits, tma, head_dim,
                               clustered=merge == "cluster" and splits in (1, 2, 4, 8))
    part_o = part_lse = counters = None
    if merge == "cluster" and splits not in (1, 2, 4, 8):
        merge = "scratch"
    if splits > 1 and merge == "scratch":
        part_o = _workspace(q.device, "decode_part_o", rows * num_heads * splits * head_dim, torch.float32)
        part_lse = _workspace(q.device, "decode_part_lse", rows * num_heads * splits, torch.float32)
        counters = _workspace(q.device, "decode_counters", rows * num_kv_heads * chunks, torch.int32)
    lib = load("attention_decode")
    _check(lib.mie_decode_attention(_ptr(q), ctypes.c_int64(q_stride), _ptr(k_cache), _ptr(v_cache),
                                    _ptr(block_tables), block_tables.shape[1], _ptr(row_q_start), _ptr(row_q_len),
                                    _ptr(row_ctx_len), rows, _ptr(out), num_heads, num_kv_heads, head_dim,
                                    page_size, ctypes.c_float(scale), int(window or 0), int(splits),
                                    _ptr(part_o), _ptr(part_lse), _ptr(counters), int(stages or 0),
                                    ctypes.c_int64(k_cache.shape[0] if tma else 0), ctypes.c_int64(k_cache.shape[0]),
                                    int(min_part_tiles if merge == "scratch" else 0),
                                    _ptr(cos), _ptr(sin), int(cos.shape[0]) if cos is not None else 0, _stream()),
           "decode_attention")
    return out


# --------------------------------------------------------------------------- activation

def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> torch.Tensor:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:]; with ``interleaved`` gate and up alternate:
    out[:, i] = silu(gate_up[:, 2i]) * gate_up[:, 2i + 1]."""
    T, two_i = gate_up.shape
    _need(two_i % 2 == 0 and out.shape == (T, two_i // 2) and out.dtype == gate_up.dtype
          and out.is_contiguous() and gate_up.is_contiguous(), "swiglu shapes/types do not match")
    lib = build.load("activation")
    _check(lib.mie_swiglu(_ptr(gate_up), _ptr(out), tag(out), T, two_i // 2, int(interleaved), _stream()), "swiglu")
    return out


# --------------------------------------------------------------------------- matrix product (CUDA cores)

def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None):
    """out[M, N] = x[M, K] @ w[N, K]^T (+ bias), float32 accumulation on CUDA cores."""
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), f"gemm shapes: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _need(x.is_contiguous() and w.is_contiguous() and out.is_contiguous(), "gemm operands must be contiguous")
    lib = build.load("gemm_simt")
    _check(lib.mie_gemm_simt(_ptr(x), tag(x), _ptr(w), tag(w), _ptr(bias), tag(bias) if bias is not None else 0,
                             _ptr(out), tag(out), M, N, K, _stream()),
           f"gemm_simt ({x.dtype}, {w.dtype} -> {out.dtype})")
    return out


# --------------------------------------------------------------------------- sampling

def sample(logits: torch.Tensor, temperature, request, position, seed: int, out: torch.Tensor,
           host_out: torch.Tensor | None = None, host_turn: torch.Tensor | None = None):
    """Token ids [rows] from float32 logits [rows, vocab]; per-row temperature (0 = greedy), request
    id (int64) and output position (int32) key the noise.  ``host_out``: a pinned host tensor
    [turns, n >= rows] int32 that also receives the tokens, in row ``host_turn[0]`` (a device int32
    tensor; row 0 without it), written by the kernel itself (pinned memory is addressable from the
    device), so that no copy has to follow."""
    rows, vocab = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "logits must be contiguous float32")
    _need(temperature.dtype == torch.float32 and request.dtype == torch.int64 and position.dtype == torch.int32
          and out.dtype == torch.int32, "sampling argument types")
    host_ptr, stride = ctypes.c_void_p(0), 0
    if host_out is not None:
        _need(host_out.dtype == torch.int32 and host_out.dim() == 2 and host_out.is_pinned() and host_out.is_contiguous()
              and host_out.shape[1] >= rows, "host_out must be a pinned int32 tensor [turns, n >= rows]")
        if host_turn is not None:
            _need(host_turn.is_cuda and host_turn.dtype == torch.int32 and host_turn.numel() >= 1, "host_turn must be a device int32 tensor")
        host_ptr, stride = ctypes.c_void_p(host_out.data_ptr()), host_out.shape[1]
    lib = build.load("sampling")
    _check(lib.mie_sample(_ptr(logits), _ptr(temperature), _ptr(request), _ptr(position),
                          ctypes.c_uint64(seed & ((1 << 64) - 1)), _ptr(out), rows, vocab, host_ptr,
                          _ptr(host_turn) if host_out is not None else ctypes.c_void_p(0), stride, _stream()), "sample")
    return out


def default_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)
