"""Integers out of range -- a token id, a position, a cache slot, a block-table entry, a gathered
row -- are reported by the kernel that meets them, and the access is skipped.

On the CPU the predicates (``csrc/range_check.cuh``, compiled for the host) are tested for their
arithmetic.  On the GPU every "out of range" value still lies INSIDE what was allocated: tables,
caches and the embedding are allocated larger than the sizes that the kernel is told, so that a
check that failed to hold could read or write only memory of this test."""
import ctypes
import math
import shutil

import pytest
import torch

TOKEN, POSITION, SLOT, PAGE, ROW = 1, 2, 3, 4, 5


@pytest.fixture(scope="module")
def predicate():
    from mini_inference_engine_b200.kernels import build
    if shutil.which("nvcc") is None and not build.os.path.isfile("/usr/local/cuda/bin/nvcc"):
        pytest.skip("no nvcc: the predicates cannot be compiled")
    lib = build.load("embedding")
    fn = lib.mie_range_predicate
    fn.argtypes = [ctypes.c_int, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong]
    return lambda kind, value, limit, limit2=0: fn(kind, value, limit, limit2)


def test_predicates_on_the_host(predicate):
    ok = 0
    # token ids: [0, vocab) or -(k+1) with k < fed-back tokens
    assert predicate(TOKEN, 0, 100, 0) == ok and predicate(TOKEN, 99, 100, 0) == ok
    assert predicate(TOKEN, 100, 100, 0) == TOKEN and predicate(TOKEN, 2 ** 31 - 1, 100, 0) == TOKEN
    assert predicate(TOKEN, -1, 100, 0) == TOKEN                       # no feedback buffer: nothing negative is valid
    assert predicate(TOKEN, -1, 100, 1) == ok and predicate(TOKEN, -8, 100, 8) == ok
    assert predicate(TOKEN, -9, 100, 8) == TOKEN and predicate(TOKEN, -2 ** 31, 100, 8) == TOKEN
    # positions
    assert predicate(POSITION, 0, 128) == ok and predicate(POSITION, 127, 128) == ok
    assert predicate(POSITION, 128, 128) == POSITION and predicate(POSITION, -1, 128) == POSITION
    # slots: pages x page size, no overflow at large pools
    assert predicate(SLOT, 16 * 10 - 1, 10, 16) == ok and predicate(SLOT, 16 * 10, 10, 16) == SLOT
    assert predicate(SLOT, -1, 10, 16) == SLOT
    assert predicate(SLOT, 2 ** 31 - 1, 2 ** 28, 128) == ok            # 2^35 slots declared: every int32 fits
    # pages and rows
    assert predicate(PAGE, 0, 5) == ok and predicate(PAGE, 4, 5) == ok and predicate(PAGE, 5, 5) == PAGE
    assert predicate(PAGE, -3, 5) == PAGE
    assert predicate(ROW, 6, 7) == ok and predicate(ROW, 7, 7) == ROW and predicate(ROW, -1, 7) == ROW


# --------------------------------------------------------------------------- on the GPU
DEV = "cuda"


@pytest.fixture()
def ops():
    from mini_inference_engine_b200.kernels import ops
    torch.cuda.synchronize()
    ops.range_report().zero_()
    yield ops
    torch.cuda.synchronize()
    ops.range_report().zero_()


def reported(ops, code, kernel, value=None, index=None):
    torch.cuda.synchronize()
    got = ops.range_report().tolist()
    assert got[0] == code and got[1] == kernel, got
    if value is not None:
        assert got[3] == value, got
    if index is not None:
        assert got[2] == index, got
    with pytest.raises(ops.KernelError, match="skipped"):
        ops.check_range_errors()
    assert ops.range_report().tolist() == [0, 0, 0, 0]                  # raising clears it
    ops.check_range_errors()


@pytest.mark.gpu
def test_embedding_reports_a_token_outside_the_vocabulary(ops):
    table = torch.randn(64, 24, device=DEV)
    feedback = torch.tensor([3, 50, 1, 2, 0, 0, 0, 0], dtype=torch.int32, device=DEV)
    ids = torch.tensor([5, 50, 39, -1], dtype=torch.int32, device=DEV)       # 50 lies in the allocation, not in the 40 declared
    out = torch.full((4, 24), 7.0, device=DEV)
    ops.embedding(table[:40], ids, out, feedback[:4])
    reported(ops, TOKEN, 1, value=50, index=1)
    assert torch.equal(out[0], table[5]) and torch.equal(out[2], table[39]) and torch.equal(out[3], table[3])
    assert (out[1] == 7.0).all()                                             # the bad row was left alone
    # a fed-back token beyond those the step declares, and a fed-back token that is itself out of range
    ops.embedding(table[:40], torch.tensor([-6], dtype=torch.int32, device=DEV), out[:1], feedback[:4])
    reported(ops, TOKEN, 1, value=-6)
    ops.embedding(table[:40], torch.tensor([-2], dtype=torch.int32, device=DEV), out[:1], feedback[:4])
    reported(ops, TOKEN, 1, value=50)


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_rotation_reports_positions_and_slots(ops, dt):
    H, Hkv, D, page, T = 4, 2, 16, 16, 3
    j = torch.arange(0, D, 2).float()
    cos, sin = ops.rope_tables((1.0 / (10000.0 ** (j / D))).to(DEV), 64)
    k_all = torch.full((8, Hkv, page, D), 7.0, dtype=dt, device=DEV)
    v_all = torch.full_like(k_all, 7.0)
    qkv0 = torch.randn(T, (H + 2 * Hkv) * D).to(dt).to(DEV)
    # position 40 is inside the 64 rows allocated and outside the 32 declared
    qkv = qkv0.clone()
    ops.rope_cache_write(qkv, torch.tensor([1, 40, 2], dtype=torch.int32, device=DEV),
                         torch.tensor([16, 17, 18], dtype=torch.int32, device=DEV), cos[:32], sin[:32], k_all[:4], v_all[:4],
                         H, Hkv, D, D, page)
    reported(ops, POSITION, 2, value=40, index=1)
    assert torch.equal(qkv[1], qkv0[1]) and not torch.equal(qkv[0], qkv0[0])
    assert (k_all[1, :, 1] == 7.0).all() and not (k_all[1, :, 0] == 7.0).all()
    # slot 5 * 16 + 3 is inside the 8 pages allocated and outside the 4 declared
    k_all.fill_(7.0)
    qkv = qkv0.clone()
    ops.rope_cache_write(qkv, torch.tensor([1, 2, 3], dtype=torch.int32, device=DEV),
                         torch.tensor([16, 5 * 16 + 3, -1], dtype=torch.int32, device=DEV), cos[:32], sin[:32], k_all[:4],
                         v_all[:4], H, Hkv, D, D, page)
    torch.cuda.synchronize()
    assert ops.range_report().tolist()[0] == SLOT and ops.range_report().tolist()[3] in (5 * 16 + 3, -1)
    ops.range_report().zero_()
    assert (k_all[4:] == 7.0).all() and (v_all[4:] == 7.0).all() and torch.equal(qkv[1], qkv0[1])


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_norm_reports_a_gathered_row_that_is_not_there(ops, dt):
    res_all = torch.randn(16, 64, device=DEV)
    delta_all = torch.randn(16, 64).to(dt).to(DEV)
    w = torch.ones(64, dtype=dt, device=DEV)
    out = torch.full((2, 64), 7.0, dtype=dt, device=DEV)
    ops.add_rmsnorm(delta_all[:8], res_all[:8], w, 1e-5, out, rows=torch.tensor([2, 11], dtype=torch.int32, device=DEV))
    reported(ops, ROW, 3, value=11, index=1)
    assert (out[1] == 7.0).all() and not (out[0] == 7.0).all()


def _attention_args(H, Hkv, D, page, ctx, q_len, bad_entry, bad_page):
    dt = torch.bfloat16
    k_all = (torch.randn(8, Hkv, page, D) * 0.5).to(dt).to(DEV)
    v_all = (torch.randn(8, Hkv, page, D) * 0.5).to(dt).to(DEV)
    q = torch.randn(q_len, H * D).to(dt).to(DEV)
    width = math.ceil(ctx / page) + 1
    bt = torch.zeros(1, width, dtype=torch.int32)
    bt[0, :width - 1] = torch.tensor([1 + (i % 3) for i in range(width - 1)])
    bt[0, bad_entry] = bad_page                       # inside the 8 pages allocated, outside the 4 declared
    meta = [torch.tensor([x], dtype=torch.int32, device=DEV) for x in (0, q_len, ctx)]
    out = torch.full((q_len, H, D), 7.0, dtype=dt, device=DEV)
    return q, k_all[:4], v_all[:4], bt.to(DEV), meta, out


@pytest.mark.gpu
@pytest.mark.parametrize("kernel,kid", [("simt", 4), ("prefill", 6), ("prefill_tc", 7)])
def test_attention_over_prompt_portions_reports_a_page_outside_the_pool(ops, kernel, kid):
    H, Hkv, D, page, ctx, q_len = 4, 2, 64, 16, 40, 40
    q, k, v, bt, (qs, ql, cl), out = _attention_args(H, Hkv, D, page, ctx, q_len, bad_entry=1, bad_page=6)
    fn = {"simt": ops.paged_attention, "prefill": ops.prefill_attention, "prefill_tc": ops.prefill_attention_tc}[kernel]
    fn(q, H * D, k, v, bt, qs, ql, cl, q_len, out, H, Hkv, D, page, 0.125, None, min_q_len=1 if kernel == "simt" else 2)
    reported(ops, PAGE, kid, value=6, index=1)
    ops.check_tc_errors()
    assert torch.isfinite(out.float()).all()         # the scratch page was read in its place


@pytest.mark.gpu
@pytest.mark.parametrize("tma", [False, True])
def test_decode_attention_reports_a_page_outside_the_pool(ops, tma):
    H, Hkv, D, page, ctx = 8, 2, 64, 16, 100
    q, k, v, bt, (qs, ql, cl), out = _attention_args(H, Hkv, D, page, ctx, 1, bad_entry=3, bad_page=5)
    ops.decode_attention(q, H * D, k, v, bt, qs, ql, cl, out, H, Hkv, D, page, 0.125, None, max_ctx=ctx, splits=2, tma=tma)
    reported(ops, PAGE, 5, value=5, index=3)
    ops.check_tc_errors()
    assert torch.isfinite(out.float()).all()


@pytest.mark.gpu
def test_simt_attention_reports_more_positions_than_the_table_covers(ops):
    H, Hkv, D, page = 4, 2, 16, 16
    q, k, v, bt, (qs, ql, cl), out = _attention_args(H, Hkv, D, page, 40, 1, bad_entry=0, bad_page=1)
    too_long = torch.tensor([bt.shape[1] * page + 1], dtype=torch.int32, device=DEV)
    ops.paged_attention(q.float(), H * D, k.float(), v.float(), bt, qs, ql, too_long, 1, out.float(), H, Hkv, D, page, 0.25)
    reported(ops, POSITION, 4, value=bt.shape[1] * page + 1, index=0)


@pytest.mark.gpu
def test_fused_projection_with_rotation_reports_positions_and_slots(ops):
    from mini_inference_engine_b200.kernels import gemm_tc
    H, Hkv, D, page, M, K = 8, 2, 64, 16, 4, 512
    N = (H + 2 * Hkv) * D
    x = (torch.randn(M, K) * 0.3).bfloat16().to(DEV)
    w = (torch.randn(N, K) * 0.05).bfloat16().to(DEV)
    assert gemm_tc.can_fuse_rope(x, w, H, Hkv, D, D)
    j = torch.arange(0, D, 2).float()
    cos, sin = ops.rope_tables((1.0 / (10000.0 ** (j / D))).to(DEV), 64)
    k_all = torch.full((8, Hkv, page, D), 7.0, dtype=torch.bfloat16, device=DEV)
    v_all = torch.full_like(k_all, 7.0)
    out = torch.full((M, N), 9.0, dtype=torch.bfloat16, device=DEV)
    positions = torch.tensor([0, 1, 45, 3], dtype=torch.int32, device=DEV)          # 45: allocated (64), not declared (32)
    slots = torch.tensor([16, 17, 18, 6 * 16], dtype=torch.int32, device=DEV)        # page 6: allocated (8), not declared (4)
    gemm_tc.gemm_qkv_rope(x, w, out, None, positions, slots, cos[:32], sin[:32], k_all[:4], v_all[:4], H, Hkv, D, D, page)
    torch.cuda.synchronize()
    gemm_tc.check_error()
    got = ops.range_report().tolist()
    assert got[1] == 8 and (got[0], got[3]) in ((POSITION, 45), (SLOT, 6 * 16)), got
    ops.range_report().zero_()
    assert (k_all[4:] == 7.0).all() and (v_all[4:] == 7.0).all()          # nothing was written beyond the declared pool
    assert (k_all[1, :, 2] == 7.0).all()                                  # nor for the token whose position was refused
    assert not (k_all[1, :, 0] == 7.0).all() and not (k_all[1, :, 1] == 7.0).all()


@pytest.mark.gpu
def test_a_step_of_the_engine_raises_on_a_report(ops, tmp_path):
    """The engine reads the report where it reads the tokens.  The report is set by hand here: a real
    batch is built by the host code whose faults the checks exist for."""
    from mini_inference_engine_b200 import EngineConfig, LLMEngine, SamplingParams
    from mini_inference_engine_b200.config import load_preset
    from mini_inference_engine_b200.weights import write_model_folder
    d = write_model_folder(str(tmp_path / "m"), load_preset("tiny-llama-a"), seed=0)
    eng = LLMEngine(d, EngineConfig(max_num_seqs=2, num_blocks=8), dtype=torch.float32, load_tokenizer=False, verbose=False)
    eng.add_request([1, 2, 3], SamplingParams(max_tokens=4, ignore_eos=True))
    eng.step()
    ops.range_report()[:] = torch.tensor([PAGE, 5, 2, 99], dtype=torch.int32)
    with pytest.raises(ops.KernelError, match="block-table entry"):
        while eng.has_work():
            eng.step()
