"""The decode-attention entry point that allocates nothing (csrc/attention_decode_static.h), called
through its exported C symbol the way a host program without an allocator would call it: inputs and
outputs only.  Its output is compared with the existing entry point's (scratch passed in by the
caller) and with the plain attention formula on two calls in a row, because the second call finds the library's scratch array as the
first one left it.  This file is collected last on purpose: if it fails, a run that stops at the
first failure has already run every other test."""
import ctypes
import math

import pytest
import torch

import plain_llama as pl
from helpers import close, scattered_tables

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(H, Hkv, D, page, ctxs, seed):
    torch.manual_seed(seed)
    num_pages = sum(math.ceil(c / page) for c in ctxs) + 2
    tables = scattered_tables(ctxs, page, num_pages, seed)
    width = max(len(t) for t in tables)
    bt = torch.zeros(len(ctxs), width, dtype=torch.int32)
    for r, t in enumerate(tables):
        bt[r, :len(t)] = torch.tensor(t)
    rows = len(ctxs)
    return dict(tables=tables, ctxs=ctxs,
        q=torch.randn(rows, H, D).bfloat16().to(DEV), k=torch.randn(num_pages, Hkv, page, D).bfloat16().to(DEV),
        v=torch.randn(num_pages, Hkv, page, D).bfloat16().to(DEV), bt=bt.to(DEV),
        q_start=torch.arange(rows, dtype=torch.int32, device=DEV), q_len=torch.ones(rows, dtype=torch.int32, device=DEV),
        ctx=torch.tensor(ctxs, dtype=torch.int32, device=DEV), H=H, Hkv=Hkv, D=D, page=page, rows=rows)


def _plain(c):
    """The newest token of every row attending to its request's keys, gathered from the pages on the host."""
    k, v, q = c["k"].float().cpu(), c["v"].float().cpu(), c["q"].float().cpu()
    out = []
    for r, (table, ctx) in enumerate(zip(c["tables"], c["ctxs"])):
        kk = torch.cat([k[p] for p in table], 1)[:, :ctx].transpose(0, 1)          # [ctx, kv_heads, D]
        vv = torch.cat([v[p] for p in table], 1)[:, :ctx].transpose(0, 1)
        qq = torch.zeros(ctx, c["H"], c["D"])
        qq[-1] = q[r]
        out.append(pl.causal_attention(qq, kk, vv, 1.0 / math.sqrt(c["D"]))[-1])
    return torch.stack(out)


def _call_static(lib, c, splits, out):
    p = lambda t: ctypes.c_void_p(t.data_ptr())      # noqa: E731
    return lib.mie_decode_attention_static(
        p(c["q"]), ctypes.c_int64(c["H"] * c["D"]), p(c["k"]), p(c["v"]), p(c["bt"]), c["bt"].shape[1], p(c["q_start"]),
        p(c["q_len"]), p(c["ctx"]), c["rows"], p(out), c["H"], c["Hkv"], c["D"], c["page"],
        ctypes.c_float(1.0 / math.sqrt(c["D"])), 0, splits, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_static_scratch_entry_point_matches_the_existing_one_twice_in_a_row():
    from mini_inference_engine_b200.kernels import build, ops
    lib = ctypes.CDLL(build.build("attention_decode_static"))
    lib.mie_decode_attention_static_error.restype = ctypes.c_char_p
    free_before = torch.cuda.mem_get_info()[0]
    for call, (shape, splits) in enumerate([((32, 4, 64, 16, [700, 33, 1, 512, 65]), 6),
                                            ((6, 3, 32, 32, [300, 90, 2000]), 9)]):
        c = _case(*shape, seed=call)
        want = torch.empty(c["rows"], c["H"], c["D"], dtype=torch.bfloat16, device=DEV)
        ops.decode_attention(c["q"], c["H"] * c["D"], c["k"], c["v"], c["bt"], c["q_start"], c["q_len"], c["ctx"], want,
                             c["H"], c["Hkv"], c["D"], c["page"], 1.0 / math.sqrt(c["D"]), splits=splits)
        got = torch.full_like(want, 99.0)
        rc = _call_static(lib, c, splits, got)
        assert rc == 0, lib.mie_decode_attention_static_error().decode()
        torch.cuda.synchronize()
        close(got, want, torch.bfloat16, f"static entry point against the existing one, call {call}")
        close(got, _plain(c), torch.bfloat16, f"static entry point against the plain formula, call {call}")
    # nothing was allocated by the entry point itself: a further call leaves free memory unchanged
    got2 = torch.full_like(want, 99.0)
    torch.cuda.synchronize()
    free_mid = torch.cuda.mem_get_info()[0]
    assert _call_static(lib, c, splits, got2) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_mid and torch.equal(got2, got)
    assert free_before >= free_mid


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from mini_inference_engine_b200.kernels import build
    lib = ctypes.CDLL(build.build("attention_decode_static"))
    lib.mie_decode_attention_static_error.restype = ctypes.c_char_p
    c = _case(32, 4, 128, 16, [40] * 64, seed=5)
    out = torch.full((64, 32, 128), 99.0, dtype=torch.bfloat16, device=DEV)
    assert _call_static(lib, c, 16, out) == -2                   # 64*32*16*128 floats > the array
    msg = lib.mie_decode_attention_static_error().decode()
    assert "too large for the static scratch" in msg and "1048576" in msg
    torch.cuda.synchronize()
    assert (out == 99.0).all()                                   # nothing was launched
    assert _call_static(lib, c, 1, out) == 0                     # one split needs no scratch
    torch.cuda.synchronize()
    assert (out != 99.0).any() and lib.mie_decode_attention_static_error() == b""
