"""The tcgen05 matrix product (``csrc/gemm_tcgen05.cu``): plan and launch.

The plan picks the orientation (weight on the 128-row side for few tokens, tokens on the 128-row
side otherwise), the tile of the other side, how far to split K so that all SMs stream, and the
depth of the shared-memory ring."""
from __future__ import annotations

import contextlib
import ctypes
import os
from dataclasses import dataclass

import torch

from . import build, ops
from .device import num_sms

SMEM_BUDGET = 226 * 1024
TWO_PER_SM = 112 * 1024


class GemmTcError(RuntimeError):
    pass


def supports(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    M, K = x.shape
    N = w.shape[0]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
            and K % 8 == 0 and N % 8 == 0 and x.is_contiguous() and w.is_contiguous() and out.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)


pdl_enabled = True      # launch with programmatic stream serialization (see csrc/gemm_tcgen05.cu)


def plan(M: int, N: int, K: int) -> dict:
    k_tiles = -(-K // 64)
    if M <= 128:
        swapped = True
        bn = next(b for b in (16, 32, 64, 128) if b >= M)
        tiles = -(-N // 128)
    else:
        swapped = False
        bn = 256 if N >= 256 else 128            # one thread issues an MMA every ~50 cycles: only 256 columns keep the tensor pipe busy
        tiles = -(-M // 128) * -(-N // bn)
    stage = 128 * 64 * 2 + bn * 64 * 2
    splits = 1
    # few tokens stream the weights, and more blocks stream faster: split up to two blocks per SM.  Many
    # tokens are bound by the tensor pipe: split only while half the SMs would otherwise idle.
    sms = num_sms()
    room = 2 * sms if swapped else sms
    while splits < 8 and tiles * splits * 2 <= room and k_tiles // (splits * 2) >= 2:
        # a cluster of 2, 4 or 8 blocks per tile, two k-tiles each at least; more blocks than SMs only if
        # each still streams four k-tiles (a second wave of short blocks costs more than it brings).  The
        # q|k|v product of TinyLlama (20 tiles, 32 k-tiles) used to run the whole decode step 11 us faster
        # with 4 splits than with 8; since a block asks L2 for its weight tiles before its dependency wait
        # the 160 blocks of 8 splits win by 6 us (0.7805 -> 0.7748 ms), and 2 splits lose 26 us
        if tiles * splits * 2 > sms and k_tiles // (splits * 2) < 4:
            break
        splits *= 2
    per_split = -(-k_tiles // splits)
    recv = 128 * (bn + 4) * 4 if swapped and splits > 1 else 0     # the slots for the peers' partial rows, beside the ring
    stages = max(2, min(8, per_split, (TWO_PER_SM - 1024 - recv) // stage))
    if stages < 3 and per_split > 2:
        stages = max(2, min(8, per_split, (SMEM_BUDGET - 1024 - recv) // stage))
    return dict(swapped=swapped, bn=bn, splits=splits, stages=stages)


@dataclass
class DeferredNorm:
    """What a product with the residual epilogue leaves for the product that reads the normed stream:
    ``xw`` = bfloat16(res * norm_weight) and, per token, sum(res^2) in ``slots`` shares.  The reader
    scales its float32 sums by rsqrt(sum / width + eps): RMSNorm without a kernel of its own
    (csrc/gemm_tcgen05.cu, the residual epilogue)."""
    xw: torch.Tensor           # [M, width] bfloat16
    sq: torch.Tensor           # [slots, M] float32
    slots: int
    width: int
    eps: float

    # enough of a tensor's face for the checks that size a product
    @property
    def shape(self):
        return self.xw.shape

    @property
    def dtype(self):
        return self.xw.dtype

    @property
    def is_cuda(self):
        return self.xw.is_cuda

    def is_contiguous(self):
        return self.xw.is_contiguous()

    def data_ptr(self):
        return self.xw.data_ptr()


class _Fuse(ctypes.Structure):
    _fields_ = [("res", ctypes.c_void_p), ("norm_w", ctypes.c_void_p), ("norm_w_tag", ctypes.c_int),
                ("xw_out", ctypes.c_void_p), ("sq_out", ctypes.c_void_p), ("sq_stride", ctypes.c_int),
                ("sq_in", ctypes.c_void_p), ("sq_slots", ctypes.c_int), ("sq_in_stride", ctypes.c_int),
                ("sq_width", ctypes.c_float), ("sq_eps", ctypes.c_float)]


def _fuse_struct(deferred: DeferredNorm | None = None, res=None, norm_weight=None, xw=None, sq=None) -> _Fuse:
    f = _Fuse()
    if res is not None:
        f.res = res.data_ptr()
        if norm_weight is not None:
            f.norm_w, f.norm_w_tag = norm_weight.data_ptr(), ops.tag(norm_weight)
            f.xw_out, f.sq_out, f.sq_stride = xw.data_ptr(), sq.data_ptr(), sq.shape[1]
    if deferred is not None:
        f.sq_in, f.sq_slots, f.sq_in_stride = deferred.sq.data_ptr(), deferred.slots, deferred.sq.shape[1]
        f.sq_width, f.sq_eps = float(deferred.width), float(deferred.eps)
    return f


# --------------------------------------------------------------------------- chains of few-token products
# csrc/gemm_chain.cu runs up to four products that follow one another in ONE launch whose blocks stay on
# their SMs and stream weights ahead through the whole chain.  The fused products of a decode step (the
# ones with the residual, norm-factor, SwiGLU and rotation epilogues) are queued here while a model runs
# its step inside ``chaining()`` and go out together: when four are queued, when any other kernel of this
# package is about to launch (ops.before_launch), or when the context ends.  Outside ``chaining()`` such a
# product is a chain of one.  Off unless MIE_B200_CHAIN=1 (or ``chain_enabled`` is set): measured on B200
# the chain loses against one launch per product at TinyLlama's sizes (see the kernel's header).

class _ChainOp(ctypes.Structure):
    _fields_ = [("x", ctypes.c_void_p), ("w", ctypes.c_void_p), ("bias", ctypes.c_void_p), ("bias_tag", ctypes.c_int),
                ("out", ctypes.c_void_p), ("N", ctypes.c_int), ("K", ctypes.c_int), ("swiglu", ctypes.c_int),
                ("positions", ctypes.c_void_p), ("slots", ctypes.c_void_p), ("cos_t", ctypes.c_void_p),
                ("sin_t", ctypes.c_void_p), ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p),
                ("num_heads", ctypes.c_int), ("num_kv_heads", ctypes.c_int), ("head_dim", ctypes.c_int),
                ("rotary_dim", ctypes.c_int), ("page_size", ctypes.c_int), ("max_pos", ctypes.c_int),
                ("write_cache", ctypes.c_int), ("num_pages", ctypes.c_longlong),
                ("res", ctypes.c_void_p), ("norm_w", ctypes.c_void_p), ("norm_w_tag", ctypes.c_int),
                ("xw_out", ctypes.c_void_p), ("sq_out", ctypes.c_void_p), ("sq_stride", ctypes.c_int),
                ("sq_in", ctypes.c_void_p), ("sq_slots", ctypes.c_int), ("sq_in_stride", ctypes.c_int),
                ("sq_width", ctypes.c_float), ("sq_eps", ctypes.c_float)]


CHAIN_MAX_TOKENS = 32
CHAIN_MAX_OPS = 4
CHAIN_SPLITS = 8
chain_enabled = os.environ.get("MIE_B200_CHAIN", "0") == "1"
_chain: list = []            # queued (op, tensors kept alive, M)
_chain_depth = 0             # > 0 inside chaining()
chain_launches = 0           # launches of the chain kernel so far, and the products they carried
chain_products = 0


def chain_takes(M: int, N: int, K: int, rope=None) -> bool:
    """Whether the chain kernel runs this fused product: few tokens; with the rotation, heads that do not
    straddle 128-row tiles and rotation partners that share an owner (every eighth row)."""
    if not chain_enabled or M < 1 or M > CHAIN_MAX_TOKENS or K % 8 or N % 8:
        return False
    if rope is not None:
        head_dim, rotary_dim = rope
        bn = 16 if M <= 16 else 32
        if head_dim <= 0 or 128 % head_dim or rotary_dim % 2 or (rotary_dim // 2) % CHAIN_SPLITS or bn * rotary_dim * 4 > 16 * 1024:
            return False
    return True


def chain_slots(N: int) -> int:
    """Shares of sum(res^2) per token that a residual epilogue of the chain kernel writes."""
    return -(-N // 128) * CHAIN_SPLITS


def flush_chain() -> None:
    """Launches what is queued, as one chain."""
    global chain_launches, chain_products
    if not _chain:
        return
    queued = list(_chain)
    _chain.clear()
    arr = (_ChainOp * len(queued))(*[q[0] for q in queued])
    lib = ops.load("gemm_chain")
    rc = lib.mie_gemm_chain(arr, len(queued), queued[0][2], 0, int(pdl_enabled), ops.raw_stream())
    ops._check(rc, f"gemm_chain of {len(queued)} products, {queued[0][2]} tokens, N x K "
               + ", ".join(f"{q[0].N} x {q[0].K}" for q in queued))
    chain_launches += 1
    chain_products += len(queued)


ops.before_launch.append(flush_chain)


@contextlib.contextmanager
def chaining():
    """Inside, fused few-token products are queued and launched as chains (see above)."""
    global _chain_depth
    _chain_depth += 1
    try:
        yield
    finally:
        _chain_depth -= 1
        if _chain_depth == 0:
            flush_chain()


def _chain_submit(x, w, bias, out, M, N, K, swiglu, fuse: "_Fuse", rope_args) -> None:
    op = _ChainOp()
    op.x, op.w, op.N, op.K, op.swiglu = x.data_ptr(), w.data_ptr(), N, K, int(swiglu)
    if bias is not None:
        op.bias, op.bias_tag = bias.data_ptr(), ops.tag(bias)
    if out is not None:
        op.out = out.data_ptr()
    keep = [x, w, bias, out]
    if rope_args is not None:
        positions, slots, cos, sin, k_cache, v_cache, H, Hkv, D, rot, page, write_cache = rope_args
        op.positions, op.slots, op.cos_t, op.sin_t = positions.data_ptr(), slots.data_ptr(), cos.data_ptr(), sin.data_ptr()
        op.k_cache, op.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
        op.num_heads, op.num_kv_heads, op.head_dim, op.rotary_dim, op.page_size = H, Hkv, D, rot, page
        op.max_pos, op.write_cache, op.num_pages = cos.shape[0], int(write_cache), k_cache.shape[0]
        keep += [positions, slots, cos, sin, k_cache, v_cache]
    for f in ("res", "norm_w", "norm_w_tag", "xw_out", "sq_out", "sq_stride", "sq_in", "sq_slots", "sq_in_stride",
              "sq_width", "sq_eps"):
        setattr(op, f, getattr(fuse, f))
    if _chain and _chain[0][2] != M:
        flush_chain()
    _chain.append((op, keep, M))
    if _chain_depth == 0 or len(_chain) == CHAIN_MAX_OPS:
        flush_chain()


def sq_slots(N: int, pl: dict) -> int:
    """Shares of sum(res^2) per token that the residual epilogue writes under plan ``pl``: one per 128-row tile and
    group of 16 or 32 rows where blocks own rows; one per tile and warp where they own tokens (tiles of 64 tokens
    and more, 4 to 16 tokens an owner)."""
    tiles = -(-N // 128)
    if pl["bn"] >= 64 and 4 <= pl["bn"] // pl["splits"] <= 16:
        return tiles * 4
    return tiles * max(pl["splits"], 4)


def splits_k(M: int, N: int, K: int) -> bool:
    """Whether the plan for these sizes puts the weight on the 128-row side and splits K across a
    cluster: the form whose owners' sum carries the rotation, residual and norm-factor epilogues."""
    pl = plan(M, N, K)
    return bool(pl["swapped"] and pl["splits"] >= 2 and -(-K // 64) >= pl["splits"] and pl["bn"] <= 128)


def _launch_fused(x, w, bias, out, M, N, K, pl, swiglu, fuse: _Fuse, rope_args=None, keep=(), chain=None):
    if chain if chain is not None else chain_takes(M, N, K, (rope_args[8], rope_args[9]) if rope_args is not None else None):
        _chain_submit(x, w, bias, out, M, N, K, swiglu, fuse, rope_args)
        if _chain:
            _chain[-1][1].extend(keep)
        return
    lib = ops.load("gemm_tcgen05")
    null = ctypes.c_void_p(0)
    if rope_args is None:
        rope_c = (null, null, null, null, null, null, 0, 0, 0, 0, 0, 0, 0, ctypes.c_longlong(0))
    else:
        positions, slots, cos, sin, k_cache, v_cache, H, Hkv, D, rot, page, write_cache = rope_args
        rope_c = (ops._ptr(positions), ops._ptr(slots), ops._ptr(cos), ops._ptr(sin), ops._ptr(k_cache), ops._ptr(v_cache),
                  H, Hkv, D, rot, page, cos.shape[0], int(write_cache), ctypes.c_longlong(k_cache.shape[0]))
    rc = lib.mie_gemm_tc_fused(ops._ptr(x), ops._ptr(w), ops._ptr(bias), ops.tag(bias) if bias is not None else 0,
                               ops._ptr(out), ops.tag(out) if out is not None else ops.tag(x), M, N, K, pl["bn"], pl["splits"],
                               pl["stages"], int(swiglu), int(pl.get("pdl", pdl_enabled)), ctypes.byref(fuse), *rope_c,
                               ops._stream())
    ops._check(rc, f"gemm_tc fused M{M} N{N} K{K} {pl}")


def gemm_residual(x, w: torch.Tensor, res: torch.Tensor, bias=None, norm_weight=None, eps: float = 0.0, **force):
    """res[M, N] += x[M, K] @ w[N, K]^T (+ bias) in place on the float32 stream ``res``.  With
    ``norm_weight`` (the RMSNorm that reads the stream next) returns the DeferredNorm for the product
    behind that norm, else None.  ``x`` may itself be a DeferredNorm.  Needs ``splits_k`` sizes."""
    deferred = x if isinstance(x, DeferredNorm) else None
    xt = deferred.xw if deferred is not None else x
    M, K = xt.shape
    N = w.shape[0]
    if (xt.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or res.dtype != torch.float32 or tuple(res.shape) != (M, N)
            or not (xt.is_contiguous() and w.is_contiguous() and res.is_contiguous()) or K % 8 or N % 8):
        raise GemmTcError(f"residual epilogue: x {tuple(xt.shape)} {xt.dtype}, w {tuple(w.shape)} {w.dtype}, "
                          f"res {tuple(res.shape)} {res.dtype} do not fit")
    pl = plan(M, N, K)
    pl.update(force)
    if not (pl["swapped"] and pl["splits"] >= 2):
        raise GemmTcError("the residual epilogue needs few tokens and a split K")
    out = None
    xw = sq = None
    chain = not force and chain_takes(M, N, K)
    if norm_weight is not None:
        slots = chain_slots(N) if chain else sq_slots(N, pl)
        xw = torch.empty(M, N, dtype=torch.bfloat16, device=res.device)
        sq = torch.empty(slots, max(M, pl["bn"] * -(-M // pl["bn"])), dtype=torch.float32, device=res.device)
        out = DeferredNorm(xw, sq, slots, N, eps)
    _launch_fused(xt, w, bias, None, M, N, K, pl, False, _fuse_struct(deferred, res, norm_weight, xw, sq),
                  keep=(res, norm_weight, xw, sq, deferred.sq if deferred is not None else None), chain=chain)
    return out


def gemm(x, w: torch.Tensor, out: torch.Tensor, bias=None, swiglu: bool = False, **force) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T (+ bias) with bfloat16 operands on tcgen05.  With ``swiglu`` the
    rows of ``w`` are gate/up interleaved and out is [M, N/2] = silu(gate) * up.  ``x`` may be a
    DeferredNorm (sizes must then satisfy ``splits_k``)."""
    deferred = x if isinstance(x, DeferredNorm) else None
    if deferred is not None:
        x = deferred.xw
    M, K = x.shape
    N = w.shape[0]
    if not supports(x, w, out) or (swiglu and N % 16):
        raise GemmTcError(f"tcgen05 gemm needs contiguous 16-byte aligned bfloat16 operands with K % 8 == 0 and "
                          f"N % 8 == 0; got x {tuple(x.shape)} {x.dtype}, w {tuple(w.shape)} {w.dtype}")
    if tuple(out.shape) != (M, N // 2 if swiglu else N):
        raise GemmTcError(f"output shape {tuple(out.shape)} does not match")
    pl = plan(M, N, K)
    pl.update(force)
    if deferred is not None:
        if not pl["swapped"]:
            raise GemmTcError("a deferred norm factor needs few tokens and a split K")
        _launch_fused(x, w, bias, out, M, N, K, pl, swiglu, _fuse_struct(deferred), keep=(deferred.sq,),
                      chain=None if not force else False)
        return out
    lib = ops.load("gemm_tcgen05")
    rc = lib.mie_gemm_tc(ops._ptr(x), ops._ptr(w), ops._ptr(bias), ops.tag(bias) if bias is not None else 0,
                         ops._ptr(out), ops.tag(out), M, N, K, int(pl["swapped"]), pl["bn"], pl["splits"], pl["stages"],
                         int(swiglu), int(pl.get("pdl", pdl_enabled)), ops._stream())
    ops._check(rc, f"gemm_tc M{M} N{N} K{K} {pl}")
    return out


def can_fuse_rope(x: torch.Tensor, w: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                  rotary_dim: int) -> bool:
    """Whether the q|k|v projection of ``x`` can rotate and store in its epilogue: the plan must put the
    weight on the 128-row side and split K (the rotation lives in the cluster reduction), and heads
    must not straddle 128-row tiles."""
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or K % 8 or N % 8 or 128 % head_dim or rotary_dim % 2:
        return False
    if N != (num_heads + 2 * num_kv_heads) * head_dim:
        return False
    pl = plan(M, N, K)
    return (pl["swapped"] and pl["splits"] >= 2 and -(-K // 64) >= pl["splits"] and (rotary_dim // 2) % pl["splits"] == 0
            and pl["bn"] * rotary_dim * 4 <= 16 * 1024)          # the tile's cos/sin rows ride in shared memory


def gemm_qkv_rope(x, w: torch.Tensor, out: torch.Tensor, bias, positions, slots, cos, sin, k_cache, v_cache,
                  num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int, page_size: int,
                  write_cache: bool = True) -> torch.Tensor:
    """The fused q|k|v projection with rotation and cache write in the epilogue: ``out`` [M, N] gets the
    rotated q columns (the k and v columns are left unwritten); rotated k and v go to their pages.
    ``x`` may be a DeferredNorm."""
    deferred = x if isinstance(x, DeferredNorm) else None
    if deferred is not None:
        x = deferred.xw
    M, K = x.shape
    N = w.shape[0]
    if not supports(x, w, out) or not can_fuse_rope(x, w, num_heads, num_kv_heads, head_dim, rotary_dim):
        raise GemmTcError("these operands cannot take the fused rotation epilogue")
    pl = plan(M, N, K)
    pl["stages"] = min(pl["stages"], 4)      # the rotation's tables share the block's memory: a fifth stage takes it past what
                                             # lets two blocks share an SM (whole decode step 0.868 ms with four, 0.901 with five)
    if deferred is not None or chain_takes(M, N, K, (head_dim, rotary_dim)):
        _launch_fused(x, w, bias, out, M, N, K, pl, False, _fuse_struct(deferred),
                      (positions, slots, cos, sin, k_cache, v_cache, num_heads, num_kv_heads, head_dim, rotary_dim, page_size,
                       write_cache), keep=(deferred.sq,) if deferred is not None else ())
        return out
    lib = ops.load("gemm_tcgen05")
    rc = lib.mie_gemm_tc_qkv_rope(ops._ptr(x), ops._ptr(w), ops._ptr(bias), ops.tag(bias) if bias is not None else 0,
                                  ops._ptr(out), M, N, K, pl["bn"], pl["splits"], pl["stages"], int(pdl_enabled),
                                  ops._ptr(positions), ops._ptr(slots), ops._ptr(cos), ops._ptr(sin), ops._ptr(k_cache),
                                  ops._ptr(v_cache), num_heads, num_kv_heads, head_dim, rotary_dim, page_size,
                                  cos.shape[0], int(write_cache), ctypes.c_longlong(k_cache.shape[0]), ops._stream())
    ops._check(rc, f"gemm_tc_qkv_rope M{M} N{N} K{K} {pl}")
    return out


def pair_supports(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False) -> bool:
    """Whether ``gemm_pair`` takes these operands."""
    N, K = w.shape
    return (x.dtype == torch.bfloat16 == w.dtype and out.dtype in (torch.bfloat16, torch.float32) and x.is_cuda
            and K % 8 == 0 and N % (16 if swiglu else 8) == 0 and x.is_contiguous() and w.is_contiguous()
            and out.is_contiguous() and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)


def gemm_pair(x, w: torch.Tensor, out: torch.Tensor | None, bias: torch.Tensor | None = None, swiglu: bool = False,
              res: torch.Tensor | None = None, norm_weight: torch.Tensor | None = None, eps: float = 0.0):
    """out = x w^T (+ bias), or silu(gate) * value over interleaved rows of ``w`` with ``swiglu``: the product
    for many tokens on pairs of SMs (``csrc/gemm_pair_tc.cu``: 256 x 256 tiles by cta_group::2 MMAs, two
    accumulators in tensor memory, one persistent pair of blocks per two SMs).  ``x`` may be a DeferredNorm (the
    norm in front becomes a row factor on the sums).  With ``res`` (float32 [M, N]) the product is added to it
    in place instead of being written (``out`` is None); with ``norm_weight`` as well, the DeferredNorm for the
    product behind that norm is returned."""
    deferred = x if isinstance(x, DeferredNorm) else None
    xt = deferred.xw if deferred is not None else x
    M, K = xt.shape
    N = w.shape[0]
    probe = out if out is not None else xt
    if not pair_supports(xt, w, probe, swiglu) or w.shape[1] != K:
        raise GemmTcError(f"gemm_pair: x {tuple(xt.shape)} {xt.dtype}, w {tuple(w.shape)} {w.dtype}")
    lib = ops.load("gemm_pair_tc")
    made = None
    xw = sq = None
    if res is not None:
        if out is not None or swiglu or res.dtype != torch.float32 or tuple(res.shape) != (M, N) or not res.is_contiguous():
            raise GemmTcError(f"gemm_pair into the stream: res {tuple(res.shape)} {res.dtype} for a product of {(M, N)}")
        if norm_weight is not None:
            slots = lib.mie_gemm_pair_slots(N)
            xw = torch.empty(M, N, dtype=torch.bfloat16, device=res.device)
            sq = torch.empty(slots, M, dtype=torch.float32, device=res.device)
            made = DeferredNorm(xw, sq, slots, N, eps)
    elif out is None or tuple(out.shape) != (M, N // 2 if swiglu else N):
        raise GemmTcError(f"gemm_pair: out {None if out is None else tuple(out.shape)} for a product of {(M, N)}")
    fuse = _fuse_struct(deferred, res, norm_weight, xw, sq)
    ops._check(lib.mie_gemm_pair(ops._ptr(xt), ops._ptr(w), ops._ptr(bias), ops.tag(bias) if bias is not None else 0,
                                 ops._ptr(out), ops.tag(out) if out is not None else 0, M, N, K, int(swiglu),
                                 ctypes.byref(fuse), ops._stream()), "gemm_pair")
    return made if res is not None else out


def check_error() -> None:
    """Raises if a block of an earlier launch gave up a bounded wait (call after a synchronise)."""
    lib = build._libs.get("gemm_pair_tc")
    if lib is not None and lib.mie_gemm_pair_error():
        lib.mie_gemm_pair_clear_error()
        raise GemmTcError("a block of the paired product gave up waiting on a barrier; its output is not valid")
    lib = build._libs.get("gemm_chain")
    if lib is not None and lib.mie_gemm_chain_error():
        lib.mie_gemm_chain_clear_error()
        raise GemmTcError("a block of the chain kernel gave up waiting (on a barrier, on its peers or on the other "
                          "blocks); the output is not valid")
    lib = build._libs.get("gemm_tcgen05")
    if lib is None:                     # never loaded: nothing was launched
        return
    if lib.mie_gemm_tc_error():
        lib.mie_gemm_tc_clear_error()
        raise GemmTcError("a tcgen05 gemm block gave up waiting on a barrier; its output is not valid")
