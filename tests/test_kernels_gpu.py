"""Each CUDA kernel alone against the plain float32 formulas, at sizes other than the engine's."""
import math
import random

import pytest
import torch

import plain_llama as pl
from helpers import close, scattered_tables

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from mini_inference_engine_b200.kernels import ops
    return ops


@pytest.mark.parametrize("tdt", DTYPES)
def test_embedding(ops, tdt):
    torch.manual_seed(0)
    table = torch.randn(301, 100).to(tdt).to(DEV)
    ids = torch.tensor([0, 300, 7, 7, 150], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 100, device=DEV)
    ops.embedding(table, ids, out)
    assert torch.equal(out.cpu(), pl.embedding(table.cpu(), ids.cpu()))


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("rows,n", [(1, 96), (7, 2048), (256, 896), (3, 11000), (5, 1)])
def test_add_rmsnorm(ops, dt, rows, n):
    torch.manual_seed(rows + n)
    delta = torch.randn(rows, n).to(dt).to(DEV)
    res = torch.randn(rows, n, device=DEV) * 3
    w = (1 + 0.1 * torch.randn(n)).to(dt).to(DEV)
    want_res = res.cpu() + delta.float().cpu()
    want = pl.rmsnorm(want_res, w.cpu(), 1e-5)
    out = torch.empty(rows, n, dtype=dt, device=DEV)
    res2 = res.clone()
    ops.add_rmsnorm(delta, res2, w, 1e-5, out)
    assert torch.equal(res2.cpu(), want_res)              # the residual sum is exact float32
    close(out, want, dt, "norm")
    # no delta (first layer): residual untouched
    res3 = res.clone()
    ops.add_rmsnorm(None, res3, w, 1e-5, out)
    assert torch.equal(res3, res)
    close(out, pl.rmsnorm(res.cpu(), w.cpu(), 1e-5), dt, "norm without delta")
    # float32 weight beside bfloat16 activations stays float32
    ops.add_rmsnorm(delta, res.clone(), w.float(), 1e-5, out)
    close(out, want, dt, "norm with float32 weight")


@pytest.mark.parametrize("dt", DTYPES)
def test_add_rmsnorm_gathers_rows_and_leaves_the_residual(ops, dt):
    torch.manual_seed(3)
    delta = torch.randn(9, 200).to(dt).to(DEV)
    res = torch.randn(9, 200, device=DEV)
    w = torch.randn(200).to(dt).to(DEV)
    rows = torch.tensor([8, 0, 3, 3], dtype=torch.int32, device=DEV)
    out = torch.empty(4, 200, dtype=dt, device=DEV)
    before = res.clone()
    ops.add_rmsnorm(delta, res, w, 1e-6, out, rows)
    assert torch.equal(res, before)
    want = pl.rmsnorm((before.cpu() + delta.float().cpu())[rows.cpu().long()], w.cpu(), 1e-6)
    close(out, want, dt, "gathered norm")


@pytest.mark.parametrize("theta,rot,max_pos", [(10000.0, 16, 128), (500000.0, 48, 5000), (1e6, 128, 3000)])
def test_rope_tables(ops, theta, rot, max_pos):
    j = torch.arange(0, rot, 2, dtype=torch.int64).float()
    inv = 1.0 / (theta ** (j / rot))
    cos, sin = ops.rope_tables(inv.to(DEV), max_pos)
    ang = pl.rope_angles(torch.arange(max_pos), rot, theta)
    # angles reach thousands of radians: float32 sin/cos of the same float32 angle
    assert (cos.cpu() - ang.cos()).abs().max() < 2e-6 and (sin.cpu() - ang.sin()).abs().max() < 2e-6


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("H,Hkv,D,rot,page", [(4, 2, 16, 16, 16), (3, 1, 48, 48, 32), (8, 8, 128, 64, 16), (5, 5, 32, 0, 64)])
def test_rope_and_cache_write(ops, dt, H, Hkv, D, rot, page):
    torch.manual_seed(H * D)
    T, theta, max_pos, num_pages = 11, 10000.0, 512, 12
    qkv = torch.randn(T, (H + 2 * Hkv) * D).to(dt)
    positions = torch.tensor([0, 1, 2, 15, 16, 17, 100, 333, 31, 32, 511], dtype=torch.int32)
    slots = torch.randperm((num_pages - 1) * page)[:T].to(torch.int32) + page       # never the scratch page
    if rot:
        j = torch.arange(0, rot, 2, dtype=torch.int64).float()
        cos, sin = ops.rope_tables((1.0 / (theta ** (j / rot))).to(DEV), max_pos)
    else:
        cos = sin = torch.zeros(max_pos, 0, device=DEV)
    k_cache = torch.full((num_pages, Hkv, page, D), 7.0, dtype=dt, device=DEV)
    v_cache = torch.full_like(k_cache, 7.0)
    dev_qkv = qkv.to(DEV)
    ops.rope_cache_write(dev_qkv, positions.to(DEV), slots.to(DEV), cos, sin, k_cache, v_cache, H, Hkv, D, rot, page)
    q, k, v = qkv.float().split([H * D, Hkv * D, Hkv * D], -1)
    q, k, v = q.view(T, H, D), k.view(T, Hkv, D), v.view(T, Hkv, D)

    def rotate(x):
        if not rot:
            return x
        ang = pl.rope_angles(positions, rot, theta)
        return torch.cat((pl.apply_rope(x[..., :rot], ang), x[..., rot:]), -1)

    close(dev_qkv[:, :H * D].reshape(T, H, D), rotate(q), dt, "rotated q")
    assert torch.equal(dev_qkv[:, H * D:].cpu(), qkv[:, H * D:])          # k, v in the activation are untouched
    kc, vc = k_cache.cpu().float(), v_cache.cpu().float()
    want_k = rotate(k)
    for t in range(T):
        pg, off = int(slots[t]) // page, int(slots[t]) % page
        close(kc[pg, :, off], want_k[t], dt, f"cached k of token {t}")
        assert torch.equal(vc[pg, :, off], v[t].to(dt).float())
    untouched = torch.ones(num_pages * page, dtype=torch.bool)
    untouched[slots.long()] = False
    assert (kc.permute(0, 2, 1, 3).reshape(num_pages * page, -1)[untouched] == 7.0).all()   # nothing else was written


def _paged_case(ops, dt, H, Hkv, D, page, rows, window=None, seed=0, boost=None, kernel="simt", min_q_len=1, work=None):
    """rows: list of (q_len, ctx_len).  Builds random q/k/v per request, scatters k/v into pages, runs
    the kernel and the plain attention on each request's whole sequence."""
    torch.manual_seed(seed)
    num_pages = sum(math.ceil(c / page) for _, c in rows) + 3
    tables = scattered_tables([c for _, c in rows], page, num_pages, seed)
    width = max(len(t) for t in tables) + 1
    k_cache = (torch.randn(num_pages, Hkv, page, D) * 3).to(dt)        # stale junk everywhere, finite
    v_cache = (torch.randn(num_pages, Hkv, page, D) * 3).to(dt)
    q_all, want = [], []
    scale = 1.0 / math.sqrt(D)
    for r, (ql, cl) in enumerate(rows):
        q = torch.randn(cl, H, D).to(dt)
        k = torch.randn(cl, Hkv, D).to(dt)
        v = torch.randn(cl, Hkv, D).to(dt)
        if boost is not None:                                         # one far key must dominate the last query
            key = boost if boost < cl else 0
            k[key] *= 0
            k[key, :, 0] = 30.0
            q[-1] *= 0
            q[-1, :, 0] = 30.0
            v[key] = 5.0
        for p in range(cl):
            k_cache[tables[r][p // page], :, p % page] = k[p]
            v_cache[tables[r][p // page], :, p % page] = v[p]
        q_all.append(q[cl - ql:])
        want.append(pl.causal_attention(q.float(), k.float(), v.float(), scale, window)[cl - ql:])
    q_all = torch.cat(q_all, 0)
    T = q_all.shape[0]
    bt = torch.zeros(len(rows), width, dtype=torch.int32)
    for r, t in enumerate(tables):
        bt[r, :len(t)] = torch.tensor(t)
        bt[r, len(t):] = 0
    q_len = torch.tensor([a for a, _ in rows], dtype=torch.int32)
    ctx_len = torch.tensor([c for _, c in rows], dtype=torch.int32)
    q_start = torch.cumsum(q_len, 0, dtype=torch.int32) - q_len
    out = torch.full((T, H, D), 77.0, dtype=dt, device=DEV)
    fn = {"simt": ops.paged_attention, "prefill": ops.prefill_attention, "prefill_tc": ops.prefill_attention_tc}[kernel]
    more = {} if work is None else {"work": work}
    fn(q_all.to(DEV).contiguous(), H * D, k_cache.to(DEV), v_cache.to(DEV), bt.to(DEV), q_start.to(DEV),
       q_len.to(DEV), ctx_len.to(DEV), T, out, H, Hkv, D, page, scale, window, min_q_len=min_q_len, **more)
    torch.cuda.synchronize()
    ops.check_tc_errors()
    return out, torch.cat(want, 0)


RAGGED = [[(1, 1)], [(1, 17)], [(1, 1000)], [(1, 2048)],
          [(1, 5), (1, 300), (1, 1), (1, 2047), (1, 64), (1, 65)],            # decode rows, the reference's ragged case
          [(5, 5), (17, 17), (33, 33)],                                       # whole prompts
          [(7, 40), (2, 18), (1, 129), (16, 16), (31, 300)],                  # continued portions beside decodes
          [(300, 300)]]


@pytest.mark.parametrize("kernel,D", [("prefill_tc", 64), ("prefill_tc", 128), ("prefill", 48), ("simt", 32)])
@pytest.mark.parametrize("hint", [False, True])
def test_portions_among_hundreds_of_one_token_rows(ops, kernel, D, hint):
    """A step of many decoding requests and a few prompt portions: the kernels for portions find a block's row among
    hundreds of rows that are not theirs (32 rows a round, by a whole warp), in front of, between and behind the
    portions; with the caller's count of portions and their tokens the launch has no blocks for the others (and must
    still reach every tile), without it the surplus blocks leave at once.  One-token rows stay untouched by the
    kernels that skip them."""
    rng = random.Random(D)
    rows = ([(1, rng.randrange(1, 80)) for _ in range(70)] + [(200, 260)] + [(1, rng.randrange(1, 80)) for _ in range(100)]
            + [(2, 2), (129, 129)] + [(1, rng.randrange(1, 80)) for _ in range(90)] + [(300, 300)] + [(1, 5)] * 3)
    min_q_len = 1 if kernel == "simt" else 2
    long = [q for q, _ in rows if q >= min_q_len]
    out, want = _paged_case(ops, torch.bfloat16, 8, 2, D, 16, rows, kernel=kernel, min_q_len=min_q_len, seed=D,
                            work=(len(long), sum(long)) if hint and kernel != "simt" else None)
    q_len = torch.tensor([q for q, _ in rows])
    live = torch.repeat_interleave(q_len >= min_q_len, q_len)
    close(out[live.to(DEV)], want[live], torch.bfloat16, f"{kernel}: portions among one-token rows")
    assert (out[~live.to(DEV)] == 77.0).all()


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("rows", RAGGED)
def test_paged_attention_ragged(ops, dt, rows):
    out, want = _paged_case(ops, dt, 32, 4, 64, 16, rows)
    close(out, want, dt, f"attention rows {rows}")


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("H,Hkv,D,page", [(4, 2, 16, 16), (3, 1, 32, 16), (6, 6, 48, 32), (16, 1, 128, 64),
                                          (2, 1, 256, 16), (12, 4, 80, 128), (40, 2, 16, 16)])
def test_paged_attention_head_shapes(ops, dt, H, Hkv, D, page):
    out, want = _paged_case(ops, dt, H, Hkv, D, page, [(1, 70), (9, 41), (35, 35), (2, 2)], seed=H + D)
    close(out, want, dt, f"attention H{H} Hkv{Hkv} D{D} page{page}")


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("window", [1, 5, 16, 33, 100])
def test_paged_attention_window_edges(ops, dt, window):
    out, want = _paged_case(ops, dt, 4, 2, 32, 16, [(1, 90), (20, 60), (50, 50), (1, 3)], window=window, seed=window)
    close(out, want, dt, f"attention window {window}")


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("far", [0, 15, 16, 511, 777])
def test_paged_attention_one_far_key_among_hundreds(ops, dt, far):
    """The last query's score for key `far` stands out: the output must be that key's value, so a
    kernel that skips or misplaces one key (a page edge, a tile edge) cannot hide behind the average."""
    out, want = _paged_case(ops, dt, 8, 2, 64, 16, [(1, 800), (3, 800)], boost=far, seed=far)
    assert (want[0] - 5.0).abs().max() < 1e-3
    close(out, want, dt, f"far key {far}")


def test_paged_attention_refuses_head_sizes_it_does_not_take(ops):
    from mini_inference_engine_b200.kernels.ops import KernelError
    z = torch.zeros(1, 1, 24, device=DEV)
    i = torch.zeros(1, 1, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError, match="head_dim"):
        ops.paged_attention(z, 24, z, z, i, i[0], i[0], i[0], 1, z.clone(), 1, 1, 24, 16, 1.0)


@pytest.mark.parametrize("dt", DTYPES)
def test_swiglu(ops, dt):
    torch.manual_seed(1)
    gu = (torch.randn(13, 2 * 176) * 3).to(dt).to(DEV)
    out = torch.empty(13, 176, dtype=dt, device=DEV)
    ops.swiglu(gu, out)
    close(out, pl.swiglu(gu.cpu()[:, :176], gu.cpu()[:, 176:]), dt, "swiglu")


@pytest.mark.parametrize("types", [(torch.float32, torch.float32, torch.float32),
                                   (torch.bfloat16, torch.bfloat16, torch.bfloat16),
                                   (torch.bfloat16, torch.bfloat16, torch.float32),
                                   (torch.bfloat16, torch.float32, torch.bfloat16),
                                   (torch.bfloat16, torch.float32, torch.float32)])
@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (3, 384, 176), (8, 2048, 96), (17, 100, 2048), (70, 130, 50),
                                   (200, 256, 64), (300, 384, 176), (260, 129, 33)])
def test_gemm_simt(ops, types, M, N, K):
    xt, wt, yt = types
    torch.manual_seed(M * N + K)
    x = torch.randn(M, K).to(xt).to(DEV)
    w = torch.randn(N, K).to(wt).to(DEV)
    b = torch.randn(N).to(wt).to(DEV)
    y = torch.empty(M, N, dtype=yt, device=DEV)
    want = (x.double().cpu() @ w.double().cpu().t())
    ops.gemm_simt(x, w, y)
    close(y, want.float(), yt, "gemm")
    if yt == torch.float32:                                 # float32 result: float32 accuracy whatever the inputs
        assert (y.cpu().double() - want).abs().max() <= 1e-5 * max(1.0, want.abs().max())
    ops.gemm_simt(x, w, y, b)
    close(y, (want + b.double().cpu()).float(), yt, "gemm + bias")


def test_sampling_greedy_and_ties(ops):
    lg = torch.zeros(3, 1000, device=DEV)
    lg[0, 999] = 1.0
    lg[1, [17, 500]] = 2.0                                  # a tie: the lowest index wins
    lg[2] = -torch.arange(1000.0)
    out = torch.empty(3, dtype=torch.int32, device=DEV)
    z = torch.zeros(3, device=DEV)
    ops.sample(lg, z, torch.zeros(3, dtype=torch.int64, device=DEV), torch.zeros(3, dtype=torch.int32, device=DEV), 0, out)
    assert out.tolist() == [999, 17, 0]
    # a large vocabulary is cut into slices, one block each: ties across slices, winners in the first
    # and the last slice, rows that are not 16-byte aligned (odd vocabulary)
    for vocab in (32000, 32003, 4099):
        lg = torch.zeros(5, vocab, device=DEV)
        lg[0, vocab - 1] = 1.0
        lg[1, [4001, vocab - 50, vocab - 2]] = 2.0             # all inside the smallest vocabulary here
        lg[2] = -torch.arange(float(vocab))
        lg[3, vocab // 2 + 1] = 0.5
        lg[4] = torch.arange(float(vocab)) % 7                  # the first 6 is at index 6
        out = torch.empty(5, dtype=torch.int32, device=DEV)
        ops.sample(lg, torch.zeros(5, device=DEV), torch.zeros(5, dtype=torch.int64, device=DEV),
                   torch.zeros(5, dtype=torch.int32, device=DEV), 0, out)
        assert out.tolist() == [vocab - 1, 4001, 0, vocab // 2 + 1, 6], vocab


@pytest.mark.parametrize("vocab", [384, 5000, 32000, 32003])
def test_sampling_temperature_matches_plain(ops, vocab):
    torch.manual_seed(vocab)
    rows = 6
    lg = torch.randn(rows, vocab) * 2
    temps = torch.tensor([0.8, 0.0, 1.5, 0.8, 0.1, 1.0])
    req = torch.tensor([3, 3, 2 ** 40 + 5, 4, 0, 77], dtype=torch.int64)
    pos = torch.tensor([0, 1, 2, 0, 9, 5], dtype=torch.int32)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops.sample(lg.to(DEV), temps.to(DEV), req.to(DEV), pos.to(DEV), 1234, out)
    for r in range(rows):
        tok = int(out[r])
        if temps[r] == 0:
            assert tok == int(lg[r].argmax())
            continue
        scores = pl.sample_scores(lg[r], float(temps[r]), 1234, int(req[r]), int(pos[r]))
        # the kernel's token is the plain argmax, or ties with it within float32 rounding of log()
        assert scores[tok] >= scores.max() - 1e-4 * max(1.0, scores.abs().max())
    # the same request and position give the same token in another batch order
    out2 = torch.empty(rows, dtype=torch.int32, device=DEV)
    perm = torch.tensor([5, 4, 3, 2, 1, 0])
    ops.sample(lg[perm].to(DEV), temps[perm].to(DEV), req[perm].to(DEV), pos[perm].to(DEV), 1234, out2)
    assert out2.cpu()[perm.argsort()].tolist() == out.tolist()


# --------------------------------------------------------------------------- tensor-core decode attention

def _decode_case(ops, H, Hkv, D, page, ctxs, splits, window=None, seed=0, boost=None, q_lens=None, max_ctx=None,
                 merge="cluster", min_part_tiles=0):
    """Rows with one new token each (or q_lens given: rows with more are to be skipped)."""
    dt = torch.bfloat16
    torch.manual_seed(seed)
    q_lens = q_lens or [1] * len(ctxs)
    num_pages = sum(math.ceil(c / page) for c in ctxs) + 3
    tables = scattered_tables(ctxs, page, num_pages, seed)
    width = max(len(t) for t in tables) + 2
    k_cache = (torch.randn(num_pages, Hkv, page, D) * 3).to(dt)
    v_cache = (torch.randn(num_pages, Hkv, page, D) * 3).to(dt)
    q_all, want = [], []
    scale = 1.0 / math.sqrt(D)
    for r, (ql, cl) in enumerate(zip(q_lens, ctxs)):
        q = torch.randn(cl, H, D).to(dt)
        k = torch.randn(cl, Hkv, D).to(dt)
        v = torch.randn(cl, Hkv, D).to(dt)
        if boost is not None:
            key = boost if boost < cl else 0
            k[key] *= 0
            k[key, :, 0] = 30.0
            q[-1] *= 0
            q[-1, :, 0] = 30.0
            v[key] = 5.0
        for p in range(cl):
            k_cache[tables[r][p // page], :, p % page] = k[p]
            v_cache[tables[r][p // page], :, p % page] = v[p]
        q_all.append(q[cl - ql:])
        want.append(pl.causal_attention(q.float(), k.float(), v.float(), scale, window)[cl - ql:])
    q_all = torch.cat(q_all, 0)
    T = q_all.shape[0]
    bt = torch.zeros(len(ctxs), width, dtype=torch.int32)
    for r, t in enumerate(tables):
        bt[r, :len(t)] = torch.tensor(t)
    q_len = torch.tensor(q_lens, dtype=torch.int32)
    ctx_len = torch.tensor(ctxs, dtype=torch.int32)
    q_start = torch.cumsum(q_len, 0, dtype=torch.int32) - q_len
    args = (q_all.to(DEV).contiguous(), H * D, k_cache.to(DEV), v_cache.to(DEV), bt.to(DEV),
            q_start.to(DEV), q_len.to(DEV), ctx_len.to(DEV))
    out = torch.full((T, H, D), 77.0, dtype=dt, device=DEV)
    ops.decode_attention(*args, out, H, Hkv, D, page, scale, window, max_ctx=max_ctx or max(ctxs), splits=splits, merge=merge,
                         tma=False, min_part_tiles=min_part_tiles)
    if D in (64, 128) and page >= 8:
        # the same case with keys and values fetched a page per TMA copy (the wrapper picks that way only
        # for many blocks): both ways must give the answer, skipped rows untouched in both
        out_tma = torch.full((T, H, D), 77.0, dtype=dt, device=DEV)
        ops.decode_attention(*args, out_tma, H, Hkv, D, page, scale, window, max_ctx=max_ctx or max(ctxs), splits=splits,
                             merge=merge, tma=True, min_part_tiles=min_part_tiles)
        torch.cuda.synchronize()
        ops.check_tc_errors()
        live = torch.repeat_interleave(q_len == 1, q_len).to(DEV)
        close(out_tma[live], torch.cat(want, 0)[live.cpu()], dt, f"decode attention by TMA, H{H} Hkv{Hkv} D{D} page{page} ctx {ctxs[:6]}")
        assert (out_tma[~live] == 77.0).all()
    return out, torch.cat(want, 0), q_start.tolist()


@pytest.mark.parametrize("merge", ["cluster", "scratch"])
@pytest.mark.parametrize("splits", [2, 4, 8])
def test_decode_attention_merges_through_cluster_or_scratch(ops, splits, merge):
    for shape in ((32, 4, 64, 16), (16, 1, 128, 16), (6, 2, 48, 32)):
        out, want, _ = _decode_case(ops, *shape, [700, 33, 1, 512, 65, 2048], splits, merge=merge, seed=splits)
        close(out, want, torch.bfloat16, f"decode {shape} splits {splits} merged by {merge}")


@pytest.mark.parametrize("splits", [None, 1, 3, 8])
@pytest.mark.parametrize("ctxs", [[1], [17], [1000], [2048], [5, 300, 1, 2047, 64, 65], list(range(1, 200, 7))])
def test_decode_attention_ragged_contexts_and_splits(ops, ctxs, splits):
    """The reference's own cases (tests/test_kernels.py:45-59 of the reference): ragged contexts, 1 / 3 / 8
    splits, and a looser static bound as under captured graphs."""
    out, want, _ = _decode_case(ops, 32, 4, 64, 16, ctxs, splits)
    close(out, want, torch.bfloat16, f"decode ctx {ctxs[:6]} splits {splits}")
    if splits is None:
        out, want, _ = _decode_case(ops, 32, 4, 64, 16, ctxs, None, max_ctx=2048)
        close(out, want, torch.bfloat16, "decode with a static context bound")


@pytest.mark.parametrize("splits,part_tiles", [(2, 8), (5, 2), (9, 1), (16, 4), (3, 0)])
def test_decode_attention_cuts_each_row_by_its_own_length(ops, splits, part_tiles):
    """A launch laid out for long contexts (scratch merge, any number of parts): a row is cut into at most
    (its 64-key tiles / part_tiles) parts, the blocks of the other parts leave at once, a row that stays whole
    writes its output itself.  Lengths around the tile and part edges; twice on the same scratch, because the
    counters of a unit are reset by the part that finds it complete -- whatever number that was."""
    ctxs = [1, 63, 64, 65, 127, 128, 129, 511, 512, 513, 700, 1023, 1024, 1025, 2048, 3000]
    for turn in range(2):
        out, want, _ = _decode_case(ops, 8, 2, 64, 16, ctxs, splits, merge="scratch", min_part_tiles=part_tiles, max_ctx=4096,
                                    seed=splits + turn)
        close(out, want, torch.bfloat16, f"decode, {splits} parts of {part_tiles} tiles or more, turn {turn}")
    out, want, _ = _decode_case(ops, 6, 3, 128, 32, ctxs[5:], splits, merge="scratch", min_part_tiles=part_tiles, max_ctx=4096,
                                window=600, seed=splits)
    close(out, want, torch.bfloat16, f"decode with a window, {splits} parts of {part_tiles} tiles or more")


def test_decode_attention_plan_for_long_contexts(ops):
    """The plan the wrapper makes by itself for 64 and more (row, kv head) units under a long context bound
    (parts through scratch, rows cut by their own lengths) gives the plain answer, ragged lengths included."""
    from mini_inference_engine_b200.kernels import ops as ops_mod
    assert ops_mod.decode_plan(24, 4, 8192, True) == (6, "scratch", ops_mod.LONG_PART_TILES)
    ctxs = [3000, 17, 1, 512, 513, 2048, 100, 1024] * 3
    out, want, _ = _decode_case(ops, 32, 4, 64, 16, ctxs, None, merge=None, max_ctx=8192, seed=3)
    close(out, want, torch.bfloat16, "decode, planned for 8,192 keys")
    # and where a cluster cuts as often as scratch would, the cluster of the plan (4 parts, page copies by TMA)
    assert ops_mod.decode_plan(32, 4, 8192, True) == (4, "cluster", 0)
    ctxs = [3000, 17, 1, 512, 513, 2048, 100, 1024] * 4
    out, want, _ = _decode_case(ops, 32, 4, 64, 16, ctxs, None, merge=None, max_ctx=8192, seed=4)
    close(out, want, torch.bfloat16, "decode, planned for 8,192 keys, 32 rows")


@pytest.mark.parametrize("H,Hkv,D,page", [(4, 2, 16, 16), (3, 1, 32, 16), (6, 6, 48, 32), (16, 1, 128, 64),
                                          (12, 4, 80, 128), (40, 2, 16, 16), (34, 1, 64, 16), (8, 8, 112, 16)])
def test_decode_attention_head_shapes(ops, H, Hkv, D, page):
    for splits in (1, 4):
        out, want, _ = _decode_case(ops, H, Hkv, D, page, [70, 41, 300, 2, 129], splits, seed=H + D)
        close(out, want, torch.bfloat16, f"decode H{H} Hkv{Hkv} D{D} page{page} splits {splits}")


@pytest.mark.parametrize("tma", [False, True])
def test_decode_attention_reads_the_key_written_just_before_it(ops, tma):
    """The decode kernel starts copying cached keys before the kernel in front of it has finished
    (programmatic dependent launch); the newest token's key and value, which that kernel writes, must
    still be the ones it uses.  Contexts grow token by token, write and attention back to back with no
    synchronisation; every new key dominates its query, so a stale row would show in full."""
    torch.manual_seed(5)
    H, Hkv, D, page, rows, start, steps = 8, 2, 64, 16, 3, 60, 44
    pages_per_row = (start + steps + page - 1) // page
    num_pages = rows * pages_per_row + 1
    tables = torch.arange(1, num_pages, dtype=torch.int32).view(rows, pages_per_row).to(DEV)
    k_cache = (torch.randn(num_pages, Hkv, page, D) * 0.1).bfloat16().to(DEV)
    v_cache = (torch.randn(num_pages, Hkv, page, D) * 0.1).bfloat16().to(DEV)
    cos = sin = torch.zeros(4096, 0, device=DEV)
    q_start = torch.arange(rows, dtype=torch.int32, device=DEV)
    q_len = torch.ones(rows, dtype=torch.int32, device=DEV)
    outs, wants = [], []
    ins = []
    for i in range(steps):                                        # every input is on the device before the first launch
        ctx = start + i + 1
        qkv = torch.zeros(rows, (H + 2 * Hkv) * D)
        qkv[:, :H * D].view(rows, H, D)[:, :, i % D] = 30.0        # the query looks along dimension i
        qkv[:, H * D:(H + Hkv) * D].view(rows, Hkv, D)[:, :, i % D] = 30.0          # and so does the new key
        val = torch.randn(rows, Hkv, D)
        qkv[:, (H + Hkv) * D:] = val.view(rows, -1)
        slots = torch.tensor([int(tables[r, (ctx - 1) // page]) * page + (ctx - 1) % page for r in range(rows)], dtype=torch.int32)
        ins.append((qkv.bfloat16().to(DEV), torch.full((rows,), ctx - 1, dtype=torch.int32, device=DEV), slots.to(DEV),
                    torch.full((rows,), ctx, dtype=torch.int32, device=DEV)))
        wants.append(val.bfloat16().float().repeat_interleave(H // Hkv, 1))
    torch.cuda.synchronize()
    for qkv, pos, slots, ctx_len in ins:
        ops.rope_cache_write(qkv, pos, slots, cos, sin, k_cache, v_cache, H, Hkv, D, 0, page)
        out = torch.empty(rows, H * D, dtype=torch.bfloat16, device=DEV)
        ops.decode_attention(qkv, qkv.shape[1], k_cache, v_cache, tables, q_start, q_len, ctx_len, out, H, Hkv, D, page,
                             1.0 / math.sqrt(D), max_ctx=start + steps, tma=tma)
        outs.append(out)
    torch.cuda.synchronize()
    for i, (out, want) in enumerate(zip(outs, wants)):
        err = (out.float().cpu().view(rows, H, D) - want).abs().max().item()
        assert err < 0.05, f"step {i}: the newest value was not the one attended to (error {err})"


@pytest.mark.parametrize("H,Hkv,D,page", [(32, 4, 64, 16), (8, 8, 128, 16), (6, 2, 32, 32), (34, 1, 96, 16)])
@pytest.mark.parametrize("splits,merge,part_tiles", [(1, "cluster", 0), (4, "cluster", 0), (5, "scratch", 2), (None, None, 0)])
def test_decode_attention_rotates_and_writes_the_cache(ops, H, Hkv, D, page, splits, merge, part_tiles):
    """Rotation inside the decode kernel: q|k|v arrive unrotated, the cache row of the new token holds NaN.  The
    kernel must rotate q and the new key by the row's position, attend with them and leave the rotated key and the
    value in the cache -- bit for bit what the rotate-and-store kernel leaves there; skipped rows (more than one
    new token) keep their NaN.  Lengths around tile, page and part edges; the new key dominates in one row."""
    dt, theta, max_pos = torch.bfloat16, 10000.0, 2100
    torch.manual_seed(H + D + (splits or 0))
    ctxs = [1, 2, 63, 64, 65, 129, 512, 513, 700, 1024, 1025, 2048, 40]
    q_lens = [1] * (len(ctxs) - 1) + [3]
    num_pages = sum(math.ceil(c / page) for c in ctxs) + 3
    tables = scattered_tables(ctxs, page, num_pages, 1)
    width = max(len(t) for t in tables) + 2
    j = torch.arange(0, D, 2, dtype=torch.int64).float()
    cos, sin = ops.rope_tables((1.0 / (theta ** (j / D))).to(DEV), max_pos)
    k_cache = (torch.randn(num_pages, Hkv, page, D) * 3).to(dt)
    v_cache = (torch.randn(num_pages, Hkv, page, D) * 3).to(dt)
    scale = 1.0 / math.sqrt(D)
    acts, want, newest = [], [], []
    for r, (ql, cl) in enumerate(zip(q_lens, ctxs)):
        q = torch.randn(cl, H, D).to(dt)
        k = torch.randn(cl, Hkv, D).to(dt)
        v = torch.randn(cl, Hkv, D).to(dt)
        if r == 6:                                               # the new key stands out: a wrong or missing one shows in full
            k[-1] *= 6
        ang = pl.rope_angles(torch.arange(cl), D, theta)
        rq, rk = pl.apply_rope(q.float(), ang), pl.apply_rope(k.float(), ang)
        rk[:cl - ql] = rk[:cl - ql].to(dt).float()               # older keys are in the cache, rounded
        for p in range(cl - ql):
            k_cache[tables[r][p // page], :, p % page] = rk[p].to(dt)
            v_cache[tables[r][p // page], :, p % page] = v[p]
        for p in range(cl - ql, cl):                             # nothing has written the rows of the new tokens
            k_cache[tables[r][p // page], :, p % page] = float("nan")
            v_cache[tables[r][p // page], :, p % page] = float("nan")
        acts.append(torch.cat((q[cl - ql:].reshape(ql, -1), k[cl - ql:].reshape(ql, -1), v[cl - ql:].reshape(ql, -1)), 1))
        want.append(pl.causal_attention(rq, rk, v.float(), scale, None)[cl - ql:])
        newest.append((tables[r][(cl - 1) // page], (cl - 1) % page, rk[-1], v[-1]))
    qkv = torch.cat(acts, 0).to(DEV).contiguous()
    bt = torch.zeros(len(ctxs), width, dtype=torch.int32)
    for r, t in enumerate(tables):
        bt[r, :len(t)] = torch.tensor(t)
    q_len = torch.tensor(q_lens, dtype=torch.int32)
    ctx_len = torch.tensor(ctxs, dtype=torch.int32)
    q_start = torch.cumsum(q_len, 0, dtype=torch.int32) - q_len
    live = torch.repeat_interleave(q_len == 1, q_len)
    for tma in ((False, True) if D in (64, 128) else (False,)):
        kc, vc = k_cache.to(DEV), v_cache.to(DEV)
        out = torch.full((qkv.shape[0], H, D), 77.0, dtype=dt, device=DEV)
        before = qkv.clone()
        ops.decode_attention(qkv, qkv.shape[1], kc, vc, bt.to(DEV), q_start.to(DEV), q_len.to(DEV), ctx_len.to(DEV), out,
                             H, Hkv, D, page, scale, None, max_ctx=2048, splits=splits, merge=merge, tma=tma if splits else None,
                             min_part_tiles=part_tiles, rope=(cos, sin))
        torch.cuda.synchronize()
        ops.check_tc_errors()
        assert torch.equal(qkv, before)                          # the activation is read, never written
        close(out[live.to(DEV)], torch.cat(want, 0)[live], dt, f"decode with rotation inside, H{H} Hkv{Hkv} D{D} tma {tma}")
        assert (out[~live.to(DEV)] == 77.0).all()
        # the cache afterwards: the same bits as the rotate-and-store kernel writes
        kc2, vc2 = k_cache.to(DEV), v_cache.to(DEV)
        pos = torch.cat([torch.arange(c - n, c) for n, c in zip(q_lens, ctxs)]).to(torch.int32)
        slots = torch.tensor([tables[r][int(p) // page] * page + int(p) % page
                              for r, (n, c) in enumerate(zip(q_lens, ctxs)) for p in range(c - n, c)], dtype=torch.int32)
        ops.rope_cache_write(qkv.clone(), pos.to(DEV), slots.to(DEV), cos, sin, kc2, vc2, H, Hkv, D, D, page)
        for r, (pg, off, rk_new, v_new) in enumerate(newest):
            if q_lens[r] == 1:
                assert torch.equal(kc[pg, :, off], kc2[pg, :, off]) and torch.equal(vc[pg, :, off], vc2[pg, :, off]), f"row {r}"
                close(kc[pg, :, off], rk_new, dt, f"cached key of row {r}")
            else:
                assert kc[pg, :, off].isnan().all() and vc[pg, :, off].isnan().all()
        same = ~(kc.isnan() | k_cache.to(DEV).isnan())
        assert torch.equal(kc[same], k_cache.to(DEV)[same])      # nothing else was touched
    with pytest.raises(Exception, match="multiples of 32"):
        ops.decode_attention(qkv, qkv.shape[1], kc, vc, bt.to(DEV), q_start.to(DEV), q_len.to(DEV), ctx_len.to(DEV), out,
                             H, Hkv, 48, page, scale, None, max_ctx=2048, rope=(cos, sin))


@pytest.mark.parametrize("window", [1, 5, 64, 65, 100])
def test_decode_attention_window(ops, window):
    for splits in (1, 3):
        out, want, _ = _decode_case(ops, 8, 2, 32, 16, [90, 200, 3, 64, 129], splits, window=window, seed=window)
        close(out, want, torch.bfloat16, f"decode window {window} splits {splits}")


@pytest.mark.parametrize("far", [0, 15, 16, 63, 64, 511, 777, 799])
def test_decode_attention_one_far_key(ops, far):
    for splits in (1, 5):
        out, want, _ = _decode_case(ops, 8, 2, 64, 16, [800, 800], splits, boost=far, seed=far)
        assert (want[0] - 5.0).abs().max() < 1e-3
        close(out, want, torch.bfloat16, f"decode far key {far} splits {splits}")


def test_decode_attention_skips_rows_with_more_tokens_and_runs_twice(ops):
    """Rows with q_len > 1 are another kernel's: their outputs stay untouched.  A second launch on
    the same scratch gives the same answer (the split counters are left at zero)."""
    for _ in range(2):
        out, want, starts = _decode_case(ops, 8, 2, 64, 16, [100, 50, 300, 7], 4, q_lens=[1, 5, 1, 2])
        assert (out[starts[1]:starts[1] + 5] == 77.0).all() and (out[starts[3]:starts[3] + 2] == 77.0).all()
        close(out[starts[0]], want[starts[0]], torch.bfloat16, "row 0")
        close(out[starts[2]], want[starts[2]], torch.bfloat16, "row 2")


# --------------------------------------------------------------------------- tensor-core prefill attention

@pytest.mark.parametrize("rows", RAGGED + [[(2, 2), (63, 63), (64, 64), (65, 65), (129, 129)], [(2048, 2048)],
                                           [(2, 1000), (64, 1024), (100, 2047)]])
def test_prefill_attention_ragged(ops, rows):
    out, want = _paged_case(ops, torch.bfloat16, 32, 4, 64, 16, rows, kernel="prefill")
    close(out, want, torch.bfloat16, f"prefill rows {rows}")


@pytest.mark.parametrize("H,Hkv,D,page", [(4, 2, 16, 16), (3, 1, 32, 16), (6, 6, 48, 32), (16, 1, 128, 64),
                                          (12, 4, 80, 128), (5, 5, 112, 16)])
def test_prefill_attention_head_shapes(ops, H, Hkv, D, page):
    out, want = _paged_case(ops, torch.bfloat16, H, Hkv, D, page, [(1, 70), (9, 41), (135, 135), (2, 2), (70, 200)],
                            seed=H + D, kernel="prefill")
    close(out, want, torch.bfloat16, f"prefill H{H} Hkv{Hkv} D{D} page{page}")


@pytest.mark.parametrize("window", [1, 5, 16, 33, 64, 65, 100, 200])
def test_prefill_attention_window_edges(ops, window):
    out, want = _paged_case(ops, torch.bfloat16, 4, 2, 32, 16, [(1, 90), (20, 60), (150, 150), (70, 300), (2, 3)],
                            window=window, seed=window, kernel="prefill")
    close(out, want, torch.bfloat16, f"prefill window {window}")


@pytest.mark.parametrize("far", [0, 15, 16, 63, 64, 511, 777])
def test_prefill_attention_one_far_key(ops, far):
    out, want = _paged_case(ops, torch.bfloat16, 8, 2, 64, 16, [(100, 800), (3, 800)], boost=far, seed=far, kernel="prefill")
    assert (want[99] - 5.0).abs().max() < 1e-3
    close(out, want, torch.bfloat16, f"prefill far key {far}")


def test_prefill_attention_skips_single_token_rows(ops):
    out, want = _paged_case(ops, torch.bfloat16, 8, 2, 64, 16, [(1, 100), (5, 50), (1, 300), (2, 7)], kernel="prefill", min_q_len=2)
    assert (out[0] == 77.0).all() and (out[6] == 77.0).all()
    close(out[1:6], want[1:6], torch.bfloat16, "row 1")
    close(out[7:9], want[7:9], torch.bfloat16, "row 3")


# --------------------------------------------------------------------------- tcgen05 matrix product

def _tc_case(M, N, K, out_dt=torch.bfloat16, bias=False, seed=0, **force):
    from mini_inference_engine_b200.kernels import gemm_tc
    torch.manual_seed(seed + M + N + K)
    x = torch.randn(M, K).bfloat16().to(DEV)
    w = torch.randn(N, K).bfloat16().to(DEV)
    b = torch.randn(N).bfloat16().to(DEV) if bias else None
    y = torch.full((M, N), 7.0, dtype=out_dt, device=DEV)
    gemm_tc.gemm(x, w, y, b, **force)
    torch.cuda.synchronize()
    gemm_tc.check_error()
    want = x.double().cpu() @ w.double().cpu().t()
    if bias:
        want = want + b.double().cpu()
    return y, want


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (1, 2560, 2048), (8, 2048, 2048), (8, 11264, 2048), (8, 2048, 5632),
                                   (7, 264, 176), (16, 384, 96), (33, 2560, 2048), (64, 32000, 2048), (100, 1000, 200),
                                   (128, 2048, 2048)])
def test_gemm_tc_few_tokens(M, N, K):
    y, want = _tc_case(M, N, K)
    close(y, want.float(), torch.bfloat16, f"tcgen05 gemm {M}x{N}x{K}")
    y, want = _tc_case(M, N, K, out_dt=torch.float32, bias=True)
    assert (y.cpu().double() - want).abs().max() <= 2e-3 * want.abs().max()      # float32 out: only the order of sums


@pytest.mark.parametrize("M,N,K", [(129, 256, 64), (2048, 2560, 2048), (300, 384, 96), (1000, 352, 176), (512, 2048, 5632),
                                   (2048, 11264, 2048), (257, 32000, 2048)])
def test_gemm_tc_many_tokens(M, N, K):
    y, want = _tc_case(M, N, K)
    close(y, want.float(), torch.bfloat16, f"tcgen05 gemm {M}x{N}x{K}")
    y, want = _tc_case(M, N, K, out_dt=torch.float32, bias=True)
    assert (y.cpu().double() - want).abs().max() <= 2e-3 * want.abs().max()


@pytest.mark.parametrize("force", [dict(swapped=True, bn=16, splits=1, stages=2), dict(swapped=True, bn=32, splits=4, stages=3),
                                   dict(swapped=True, bn=64, splits=8, stages=8), dict(swapped=True, bn=128, splits=2, stages=4),
                                   dict(swapped=True, bn=256, splits=2, stages=4), dict(swapped=False, bn=16, splits=1, stages=4),
                                   dict(swapped=False, bn=64, splits=4, stages=6), dict(swapped=False, bn=128, splits=1, stages=3),
                                   dict(swapped=False, bn=256, splits=2, stages=4), dict(swapped=False, bn=128, splits=8, stages=2)])
@pytest.mark.parametrize("pdl", [0, 1])
def test_gemm_tc_every_tile_orientation_and_split(force, pdl):
    for M, N, K in ((40, 392, 840), (200, 520, 2048), (9, 128, 320)):       # 320 = 5 k-tiles: a split of 8 leaves blocks empty
        if force["swapped"] and M > force["bn"] * 8:
            continue
        y, want = _tc_case(M, N, K, bias=True, pdl=pdl, **force)
        close(y, want.float(), torch.bfloat16, f"tcgen05 gemm {M}x{N}x{K} {force}")
        y2, _ = _tc_case(M, N, K, bias=True, pdl=pdl, **force)          # split-K is deterministic: the same sum order every time
        assert torch.equal(y, y2)


@pytest.mark.parametrize("M,I,K,force", [(8, 5632, 2048, {}), (3, 176, 64, {}), (64, 256, 96, dict(splits=1)),
                                         (300, 176, 64, {}), (2048, 5632, 2048, {}), (40, 200, 840, dict(swapped=True, bn=64, splits=4, stages=4)),
                                         (200, 264, 2048, dict(swapped=False, bn=64, splits=4, stages=4))])
def test_gemm_tc_swiglu_epilogue(M, I, K, force):
    """gate/up rows interleaved in W; the epilogue writes silu(gate) * up from the float32 sums."""
    from mini_inference_engine_b200.kernels import gemm_tc
    torch.manual_seed(M + I)
    x = torch.randn(M, K).bfloat16()
    gate, up = (torch.randn(I, K) * 0.1).bfloat16(), (torch.randn(I, K) * 0.1).bfloat16()
    w = torch.stack((gate, up), 1).reshape(2 * I, K).contiguous()
    out = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    gemm_tc.gemm(x.to(DEV), w.to(DEV), out, swiglu=True, **force)
    torch.cuda.synchronize()
    gemm_tc.check_error()
    want = pl.swiglu(x.float() @ gate.float().t(), x.float() @ up.float().t())
    close(out, want, torch.bfloat16, f"swiglu epilogue {M}x{I}x{K}")


def test_gemm_tc_refuses_what_it_cannot_align():
    from mini_inference_engine_b200.kernels import gemm_tc
    x = torch.zeros(4, 100, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(16, 100, dtype=torch.bfloat16, device=DEV)
    assert not gemm_tc.supports(x, w, torch.zeros(4, 16, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(gemm_tc.GemmTcError):
        gemm_tc.gemm(x, w, torch.zeros(4, 16, dtype=torch.bfloat16, device=DEV))


def test_swiglu_interleaved(ops):
    torch.manual_seed(2)
    g, u = torch.randn(13, 176) * 3, torch.randn(13, 176) * 3
    gu = torch.stack((g, u), 2).reshape(13, 352).bfloat16().to(DEV)
    out = torch.empty(13, 176, dtype=torch.bfloat16, device=DEV)
    ops.swiglu(gu, out, interleaved=True)
    close(out, pl.swiglu(g.bfloat16(), u.bfloat16()), torch.bfloat16, "interleaved swiglu")


# --------------------------------------------------------------------------- tcgen05 prefill attention

@pytest.mark.parametrize("rows", [[(5, 5)], [(128, 128)], [(129, 129)], [(300, 300)], [(5, 5), (17, 17), (33, 33)],
                                  [(7, 40), (2, 18), (1, 129), (16, 16), (31, 300)], [(2, 2), (127, 127), (128, 128), (257, 257)],
                                  [(2048, 2048)], [(2, 1000), (64, 1024), (100, 2047), (200, 700)]])
def test_prefill_attention_tc_ragged(ops, rows):
    out, want = _paged_case(ops, torch.bfloat16, 32, 4, 64, 16, rows, kernel="prefill_tc")
    close(out, want, torch.bfloat16, f"tcgen05 prefill rows {rows}")


@pytest.mark.parametrize("H,Hkv,D,page", [(4, 2, 64, 16), (3, 1, 64, 32), (6, 6, 128, 16), (16, 1, 128, 64), (8, 2, 64, 128),
                                          (2, 2, 128, 8)])
def test_prefill_attention_tc_head_shapes(ops, H, Hkv, D, page):
    out, want = _paged_case(ops, torch.bfloat16, H, Hkv, D, page, [(1, 70), (9, 41), (135, 135), (2, 2), (270, 400)],
                            seed=H + D, kernel="prefill_tc")
    close(out, want, torch.bfloat16, f"tcgen05 prefill H{H} Hkv{Hkv} D{D} page{page}")


@pytest.mark.parametrize("window", [1, 5, 16, 33, 128, 129, 200])
def test_prefill_attention_tc_window_edges(ops, window):
    out, want = _paged_case(ops, torch.bfloat16, 4, 2, 64, 16, [(1, 90), (20, 60), (150, 150), (70, 300), (2, 3), (400, 400)],
                            window=window, seed=window, kernel="prefill_tc")
    close(out, want, torch.bfloat16, f"tcgen05 prefill window {window}")


@pytest.mark.parametrize("far", [0, 15, 16, 127, 128, 511, 777])
def test_prefill_attention_tc_one_far_key(ops, far):
    out, want = _paged_case(ops, torch.bfloat16, 8, 2, 64, 16, [(100, 800), (3, 800)], boost=far, seed=far, kernel="prefill_tc")
    assert (want[99] - 5.0).abs().max() < 1e-3
    close(out, want, torch.bfloat16, f"tcgen05 prefill far key {far}")


@pytest.mark.parametrize("H,Hkv,D,rows,window", [
    (32, 4, 64, [(2048, 2048)], None),                                   # 16 tiles: 8 pairs of 17 key tiles each
    (32, 4, 64, [(700, 900), (1300, 1300), (129, 500), (1, 40), (257, 257)], None),   # 6, 11, 2, 1 and 3 tiles: odd counts, a lone middle tile
    (32, 8, 64, [(1100, 1100), (900, 2000)], 300),                       # a window: the two tiles of a pair start at different keys
    (16, 2, 128, [(1500, 1500), (1000, 1200)], None),                    # head size 128: one block per SM
])
def test_prefill_attention_tc_pairs_of_query_tiles(ops, H, Hkv, D, rows, window):
    """With more query tiles than the GPU runs at a time a block takes two tiles of a row, one after
    the other (the j-th from the end and the j-th from the start), and stages and barrier phases run on
    from the first to the second.  Sizes chosen so that the launch pairs."""
    tiles = sum((q + 127) // 128 for q, _ in rows) + len(rows)
    assert tiles * H > 148 * (2 if D == 64 else 1)
    out, want = _paged_case(ops, torch.bfloat16, H, Hkv, D, 16, rows, window=window, seed=H + D, kernel="prefill_tc")
    close(out, want, torch.bfloat16, f"tcgen05 prefill in pairs, rows {rows} window {window}")


@pytest.fixture()
def side_by_side(ops):
    ops.set_prefill_pairs(1)
    yield
    ops.set_prefill_pairs(-1)


@pytest.mark.parametrize("rows,window", [
    ([(2048, 2048)], None),                                              # 8 blocks of two tiles a head
    ([(5, 5)], None), ([(128, 128)], None), ([(129, 129)], None), ([(300, 300)], None),      # one tile, two, an odd count
    ([(700, 900), (1300, 1300), (129, 500), (1, 40), (257, 257), (2, 2)], None),         # continued portions, a skipped row
    ([(1100, 1100), (900, 2000)], 300), ([(70, 300), (400, 400), (150, 150)], 33),      # windows: the second tile starts at a later key tile
    ([(400, 400)], 128), ([(400, 400)], 129), ([(513, 1200)], 1),
])
def test_prefill_attention_tc_two_query_tiles_side_by_side(ops, side_by_side, rows, window):
    """The kernel that holds two consecutive query tiles and two softmax groups a block (head_dim 64), forced for
    every launch size, against the plain formula."""
    out, want = _paged_case(ops, torch.bfloat16, 8, 2, 64, 16, rows, window=window, seed=len(rows) + (window or 0), kernel="prefill_tc",
                            min_q_len=2)
    live = torch.cat([torch.full((q,), q >= 2) for q, _ in rows])
    close(out[live], want[live], torch.bfloat16, f"two tiles side by side, rows {rows} window {window}")
    assert (out[~live] == 77.0).all()


@pytest.mark.parametrize("far", [0, 127, 128, 255, 256, 777])
@pytest.mark.parametrize("page", [16, 64, 128])
def test_prefill_attention_tc_side_by_side_one_far_key_and_page_sizes(ops, side_by_side, far, page):
    out, want = _paged_case(ops, torch.bfloat16, 8, 2, 64, page, [(300, 800), (3, 800)], boost=far, seed=far, kernel="prefill_tc")
    assert (want[299] - 5.0).abs().max() < 1e-3
    close(out, want, torch.bfloat16, f"two tiles side by side, far key {far}, page {page}")


def test_prefill_attention_tc_skips_single_token_rows(ops):
    out, want = _paged_case(ops, torch.bfloat16, 8, 2, 64, 16, [(1, 100), (5, 50), (1, 300), (2, 7)], kernel="prefill_tc", min_q_len=2)
    assert (out[0] == 77.0).all() and (out[6] == 77.0).all()
    close(out[1:6], want[1:6], torch.bfloat16, "row 1")
    close(out[7:9], want[7:9], torch.bfloat16, "row 3")


@pytest.mark.parametrize("H,Hkv,D,rot,M,K", [(32, 4, 64, 64, 8, 2048), (4, 2, 16, 16, 3, 256), (3, 1, 32, 32, 16, 384),
                                             (8, 8, 128, 64, 5, 512), (2, 1, 64, 0, 7, 256), (32, 8, 128, 128, 32, 4096),
                                             # 33 tokens and more: blocks own tokens instead of rows
                                             (32, 4, 64, 64, 64, 2048), (32, 4, 64, 64, 41, 2048), (6, 2, 32, 32, 50, 512),
                                             (8, 8, 128, 64, 64, 1024)])
def test_gemm_tc_fused_rotation_and_cache_write(ops, H, Hkv, D, rot, M, K):
    """The q|k|v product with rotation and cache write in its epilogue against the plain formulas."""
    from mini_inference_engine_b200.kernels import gemm_tc
    torch.manual_seed(H + D + M)
    N, page, num_pages, theta, max_pos = (H + 2 * Hkv) * D, 16, 40, 10000.0, 600
    x = (torch.randn(M, K) * 0.5).bfloat16()
    w = (torch.randn(N, K) * 0.05).bfloat16()
    b = (torch.randn(N) * 0.1).bfloat16()
    positions = torch.randint(0, max_pos, (M,), dtype=torch.int32)
    slots = torch.randperm((num_pages - 1) * page)[:M].to(torch.int32) + page
    if rot:
        j = torch.arange(0, rot, 2, dtype=torch.int64).float()
        cos, sin = ops.rope_tables((1.0 / (theta ** (j / rot))).to(DEV), max_pos)
    else:
        cos = sin = torch.zeros(max_pos, 0, device=DEV)
    assert gemm_tc.can_fuse_rope(x.to(DEV), w.to(DEV), H, Hkv, D, rot)
    k_cache = torch.full((num_pages, Hkv, page, D), 7.0, dtype=torch.bfloat16, device=DEV)
    v_cache = torch.full_like(k_cache, 7.0)
    out = torch.full((M, N), 9.0, dtype=torch.bfloat16, device=DEV)
    gemm_tc.gemm_qkv_rope(x.to(DEV), w.to(DEV), out, b.to(DEV), positions.to(DEV), slots.to(DEV), cos, sin, k_cache, v_cache,
                          H, Hkv, D, rot, page)
    torch.cuda.synchronize()
    gemm_tc.check_error()
    qkv = x.float() @ w.float().t() + b.float()
    q, k, v = qkv.split([H * D, Hkv * D, Hkv * D], -1)
    q, k, v = q.view(M, H, D), k.view(M, Hkv, D), v.view(M, Hkv, D)

    def rotate(t):
        if not rot:
            return t
        ang = pl.rope_angles(positions, rot, theta)
        return torch.cat((pl.apply_rope(t[..., :rot], ang), t[..., rot:]), -1)

    close(out[:, :H * D].reshape(M, H, D), rotate(q), torch.bfloat16, "fused rotated q")
    kc, vc = k_cache.cpu().float(), v_cache.cpu().float()
    for t in range(M):
        pg, off = int(slots[t]) // page, int(slots[t]) % page
        close(kc[pg, :, off], rotate(k)[t], torch.bfloat16, f"fused cached k of token {t}")
        close(vc[pg, :, off], v[t], torch.bfloat16, f"fused cached v of token {t}")
    untouched = torch.ones(num_pages * page, dtype=torch.bool)
    untouched[slots.long()] = False
    assert (kc.permute(0, 2, 1, 3).reshape(num_pages * page, -1)[untouched] == 7.0).all()
    assert (vc.permute(0, 2, 1, 3).reshape(num_pages * page, -1)[untouched] == 7.0).all()


@pytest.mark.parametrize("M,N,K", [(8, 2048, 2048), (1, 2048, 5632), (16, 2048, 5632), (13, 264, 320), (5, 1000, 840), (3, 128, 256),
                                   (64, 2048, 2048), (33, 2048, 5632), (57, 264, 512), (64, 1000, 840)])
@pytest.mark.parametrize("with_norm", [True, False])
def test_gemm_tc_residual_epilogue(M, N, K, with_norm):
    """res += x W^T + b on the float32 stream, and for the norm behind it xw = bf16(res * w_norm) and
    sum(res^2) in slots, against the plain formulas."""
    from mini_inference_engine_b200.kernels import gemm_tc
    torch.manual_seed(M + N + K)
    assert gemm_tc.splits_k(M, N, K)
    x = (torch.randn(M, K) * 0.5).bfloat16()
    w = (torch.randn(N, K) * 0.05).bfloat16()
    b = (torch.randn(N) * 0.1).bfloat16()
    res0 = torch.randn(M, N) * 2
    nw = (torch.randn(N) * 0.2 + 1).bfloat16()
    res = res0.clone().to(DEV)
    d = gemm_tc.gemm_residual(x.to(DEV), w.to(DEV), res, b.to(DEV), nw.to(DEV) if with_norm else None, 1e-5)
    torch.cuda.synchronize()
    gemm_tc.check_error()
    want = res0.double() + x.double() @ w.double().t() + b.double()
    assert (res.cpu().double() - want).abs().max() <= 1e-5 * want.abs().max() + 1e-5     # float32 sums, another order
    if not with_norm:
        assert d is None
        return
    assert d.slots == d.sq.shape[0] and d.width == N and tuple(d.xw.shape) == (M, N)
    close(d.xw, (want * nw.double()).float(), torch.bfloat16, "xw of the residual epilogue")
    sq = d.sq[:, :M].sum(0).cpu().double()
    assert ((sq - (want ** 2).sum(1)).abs() <= 1e-5 * (want ** 2).sum(1)).all()
    # every launch writes every slot: run again on junk and compare (no stale share survives)
    d.sq.fill_(1e9)
    res2 = res0.clone().to(DEV)
    d2 = gemm_tc.gemm_residual(x.to(DEV), w.to(DEV), res2, b.to(DEV), nw.to(DEV), 1e-5)
    assert torch.equal(res2, res) and torch.equal(d2.sq[:, :M], gemm_tc.gemm_residual(
        x.to(DEV), w.to(DEV), res0.clone().to(DEV), b.to(DEV), nw.to(DEV), 1e-5).sq[:, :M])


@pytest.mark.parametrize("M,h,N", [(8, 2048, 2560), (16, 2048, 11264), (3, 264, 400), (1, 2048, 2048), (64, 2048, 11264),
                                   (47, 2048, 2560), (64, 520, 400)])
@pytest.mark.parametrize("swiglu", [False, True])
def test_gemm_tc_deferred_norm_factor(ops, M, h, N, swiglu):
    """RMSNorm split across two products: the first leaves res * w and sum(res^2), the second scales its
    sums by rsqrt(mean + eps).  Together they must match norm-then-product of the plain formulas."""
    from mini_inference_engine_b200.kernels import gemm_tc
    torch.manual_seed(M + h + N)
    eps, K0 = 1e-5, 512
    a = (torch.randn(M, K0) * 0.5).bfloat16()
    w0 = (torch.randn(h, K0) * 0.05).bfloat16()
    res0 = torch.randn(M, h) * 3
    nw = (torch.randn(h) * 0.2 + 1).bfloat16()
    w1 = (torch.randn(N, h) * 0.05).bfloat16()
    b1 = None if swiglu else (torch.randn(N) * 0.1).bfloat16().to(DEV)
    assert gemm_tc.splits_k(M, h, K0) and gemm_tc.splits_k(M, N, h)
    res = res0.clone().to(DEV)
    d = gemm_tc.gemm_residual(a.to(DEV), w0.to(DEV), res, None, nw.to(DEV), eps)
    out = torch.full((M, N // 2 if swiglu else N), 9.0, dtype=torch.bfloat16, device=DEV)
    gemm_tc.gemm(d, w1.to(DEV), out, b1, swiglu=swiglu)
    torch.cuda.synchronize()
    gemm_tc.check_error()
    r = res0.double() + a.double() @ w0.double().t()
    normed = pl.rmsnorm(r.float(), nw.float(), eps).double()
    y = normed @ w1.double().t()
    if swiglu:
        want = pl.swiglu(y[:, 0::2].float(), y[:, 1::2].float())
    else:
        want = (y + b1.cpu().double()).float()
    close(out, want, torch.bfloat16, f"deferred norm factor {M}x{h}->{N} swiglu={swiglu}")


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (257, 264, 72), (2048, 2560, 2048), (300, 520, 200), (1000, 11264, 512),
                                   (33, 2048, 5632), (512, 32000, 256)])
@pytest.mark.parametrize("out_dt", [torch.bfloat16, torch.float32])
def test_gemm_pair_against_the_plain_product(M, N, K, out_dt):
    """The many-token product on pairs of SMs (256 x 256 tiles, cta_group::2): sizes that are no multiple of a
    tile in any direction, one tile and several waves of them, with a bias, against float64."""
    from mini_inference_engine_b200.kernels import gemm_tc
    torch.manual_seed(M + N + K)
    x = (torch.randn(M, K) * 0.5).bfloat16()
    w = (torch.randn(N, K) * 0.05).bfloat16()
    b = (torch.randn(N) * 0.1).bfloat16()
    out = torch.full((M, N), 9.0, dtype=out_dt, device=DEV)
    gemm_tc.gemm_pair(x.to(DEV), w.to(DEV), out, b.to(DEV))
    torch.cuda.synchronize()
    gemm_tc.check_error()
    want = (x.double() @ w.double().t() + b.double()).float()
    close(out, want, out_dt if out_dt == torch.bfloat16 else torch.float32, f"paired product {M}x{N}x{K} -> {out_dt}")


@pytest.mark.parametrize("M,N,K", [(2048, 11264, 2048), (130, 48, 96), (700, 1040, 328)])
def test_gemm_pair_swiglu(M, N, K):
    from mini_inference_engine_b200.kernels import gemm_tc
    torch.manual_seed(M + N)
    x = (torch.randn(M, K) * 0.5).bfloat16()
    w = (torch.randn(N, K) * 0.08).bfloat16()
    out = torch.full((M, N // 2), 9.0, dtype=torch.bfloat16, device=DEV)
    gemm_tc.gemm_pair(x.to(DEV), w.to(DEV), out, swiglu=True)
    torch.cuda.synchronize()
    gemm_tc.check_error()
    y = x.double() @ w.double().t()
    close(out, pl.swiglu(y[:, 0::2].float(), y[:, 1::2].float()), torch.bfloat16, f"paired product with SwiGLU {M}x{N}x{K}")


@pytest.mark.parametrize("M,h,K0,N", [(2048, 2048, 2048, 11264), (300, 264, 96, 400), (1025, 520, 200, 48)])
@pytest.mark.parametrize("swiglu", [False, True])
def test_gemm_pair_residual_and_deferred_norm(M, h, K0, N, swiglu):
    """RMSNorm split across two many-token products: the first adds to the float32 stream and leaves
    bf16(res * w_norm) and sum(res^2) per 256-column tile, the second scales its sums by rsqrt(mean + eps).
    The stream, the operand, the sums and the final product against the plain formulas."""
    from mini_inference_engine_b200.kernels import gemm_tc
    torch.manual_seed(M + h + N)
    eps = 1e-5
    a = (torch.randn(M, K0) * 0.5).bfloat16()
    w0 = (torch.randn(h, K0) * 0.05).bfloat16()
    b0 = (torch.randn(h) * 0.1).bfloat16()
    res0 = torch.randn(M, h) * 3
    nw = (torch.randn(h) * 0.2 + 1).bfloat16()
    w1 = (torch.randn(N, h) * 0.05).bfloat16()
    b1 = None if swiglu else (torch.randn(N) * 0.1).bfloat16().to(DEV)
    res = res0.clone().to(DEV)
    d = gemm_tc.gemm_pair(a.to(DEV), w0.to(DEV), None, b0.to(DEV), res=res, norm_weight=nw.to(DEV), eps=eps)
    out = torch.full((M, N // 2 if swiglu else N), 9.0, dtype=torch.bfloat16, device=DEV)
    gemm_tc.gemm_pair(d, w1.to(DEV), out, b1, swiglu=swiglu)
    torch.cuda.synchronize()
    gemm_tc.check_error()
    r = res0.double() + a.double() @ w0.double().t() + b0.double()
    assert (res.cpu().double() - r).abs().max() <= 1e-5 * r.abs().max() + 1e-5
    close(d.xw, (r * nw.double()).float(), torch.bfloat16, "operand left for the next product")
    sq = d.sq[:, :M].sum(0).cpu().double()
    assert ((sq - (r ** 2).sum(1)).abs() <= 1e-5 * (r ** 2).sum(1)).all()
    y = pl.rmsnorm(r.float(), nw.float(), eps).double() @ w1.double().t()
    want = pl.swiglu(y[:, 0::2].float(), y[:, 1::2].float()) if swiglu else (y + b1.cpu().double()).float()
    close(out, want, torch.bfloat16, f"deferred norm through paired products {M}x{h}->{N} swiglu={swiglu}")
    # without a norm behind it the stream alone is updated, and a second launch adds again
    res2 = res0.clone().to(DEV)
    assert gemm_tc.gemm_pair(a.to(DEV), w0.to(DEV), None, b0.to(DEV), res=res2) is None
    torch.cuda.synchronize()
    assert torch.equal(res2, res)


def test_gemm_tc_deferred_norm_factor_with_rotation(ops):
    """The q|k|v product with both epilogues: the norm factor first, then rotation and cache write."""
    from mini_inference_engine_b200.kernels import gemm_tc
    torch.manual_seed(11)
    H, Hkv, D, rot, M, h, page, num_pages, theta, max_pos, eps = 32, 4, 64, 64, 8, 2048, 16, 20, 10000.0, 600, 1e-5
    N = (H + 2 * Hkv) * D
    a = (torch.randn(M, 256) * 0.5).bfloat16()
    w0 = (torch.randn(h, 256) * 0.05).bfloat16()
    res0 = torch.randn(M, h) * 3
    nw = (torch.randn(h) * 0.2 + 1).bfloat16()
    w = (torch.randn(N, h) * 0.05).bfloat16()
    positions = torch.randint(0, max_pos, (M,), dtype=torch.int32)
    slots = torch.randperm((num_pages - 1) * page)[:M].to(torch.int32) + page
    j = torch.arange(0, rot, 2, dtype=torch.int64).float()
    cos, sin = ops.rope_tables((1.0 / (theta ** (j / rot))).to(DEV), max_pos)
    k_cache = torch.full((num_pages, Hkv, page, D), 7.0, dtype=torch.bfloat16, device=DEV)
    v_cache = torch.full_like(k_cache, 7.0)
    res = res0.clone().to(DEV)
    d = gemm_tc.gemm_residual(a.to(DEV), w0.to(DEV), res, None, nw.to(DEV), eps)
    out = torch.full((M, N), 9.0, dtype=torch.bfloat16, device=DEV)
    gemm_tc.gemm_qkv_rope(d, w.to(DEV), out, None, positions.to(DEV), slots.to(DEV), cos, sin, k_cache, v_cache, H, Hkv, D, rot, page)
    torch.cuda.synchronize()
    gemm_tc.check_error()
    r = res0.double() + a.double() @ w0.double().t()
    qkv = (pl.rmsnorm(r.float(), nw.float(), eps).double() @ w.double().t()).float()
    q, k, v = qkv.split([H * D, Hkv * D, Hkv * D], -1)
    ang = pl.rope_angles(positions, rot, theta)
    close(out[:, :H * D].reshape(M, H, D), pl.apply_rope(q.view(M, H, D), ang), torch.bfloat16, "rotated q behind a deferred norm")
    kc, vc = k_cache.cpu().float(), v_cache.cpu().float()
    for t in range(M):
        pg, off = int(slots[t]) // page, int(slots[t]) % page
        close(kc[pg, :, off], pl.apply_rope(k.view(M, Hkv, D), ang)[t], torch.bfloat16, f"cached k of token {t}")
        close(vc[pg, :, off], v.view(M, Hkv, D)[t], torch.bfloat16, f"cached v of token {t}")


# --------------------------------------------------------------------------- the chain kernel (off by default)

@pytest.fixture()
def chain_on():
    from mini_inference_engine_b200.kernels import gemm_tc
    before, gemm_tc.chain_enabled = gemm_tc.chain_enabled, True
    yield gemm_tc
    gemm_tc.flush_chain()
    gemm_tc.chain_enabled = before


@pytest.mark.parametrize("M", [1, 8, 13, 32])
def test_chain_of_four_products_in_one_launch(chain_on, M):
    """Output projection (residual + next norm) -> gate/up with the norm factor and SwiGLU -> down (residual + next
    norm) -> a plain product with the norm factor, queued and launched as ONE chain, against the plain formulas; at
    sizes that give blocks empty K slices (K = 320: five k-tiles for eight splits) and tiles beyond the last row."""
    gemm_tc = chain_on
    torch.manual_seed(M)
    h, I, N4 = 320, 456, 200
    attn = (torch.randn(M, h) * 0.5).bfloat16()
    Wo, Wgu = (torch.randn(h, h) * 0.05).bfloat16(), (torch.randn(2 * I, h) * 0.05).bfloat16()
    Wd, W4 = (torch.randn(h, I) * 0.05).bfloat16(), (torch.randn(N4, h) * 0.05).bfloat16()
    n1, n2 = (1 + 0.1 * torch.randn(h)).bfloat16(), (1 + 0.1 * torch.randn(h)).bfloat16()
    res0 = torch.randn(M, h)
    res = res0.clone().to(DEV)
    launches = gemm_tc.chain_launches
    with gemm_tc.chaining():
        d1 = gemm_tc.gemm_residual(attn.to(DEV), Wo.to(DEV), res, None, n1.to(DEV), 1e-5)
        act = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
        gemm_tc.gemm(d1, Wgu.to(DEV), act, swiglu=True)
        d2 = gemm_tc.gemm_residual(act, Wd.to(DEV), res, None, n2.to(DEV), 1e-5)
        out = torch.empty(M, N4, dtype=torch.bfloat16, device=DEV)
        gemm_tc.gemm(d2, W4.to(DEV), out)
    torch.cuda.synchronize()
    gemm_tc.check_error()
    assert gemm_tc.chain_launches == launches + 1
    r1 = res0 + attn.float() @ Wo.float().t()
    x1 = pl.round_bf16(r1 * n1.float())                                   # what the chain hands on: bf16(res * w)
    f1 = torch.rsqrt((r1 ** 2).mean(-1, keepdim=True) + 1e-5)
    gu = (x1 @ Wgu.float().t()) * f1
    a = pl.round_bf16(torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2])
    r2 = r1 + a @ Wd.float().t()
    x2 = pl.round_bf16(r2 * n2.float())
    f2 = torch.rsqrt((r2 ** 2).mean(-1, keepdim=True) + 1e-5)
    want = (x2 @ W4.float().t()) * f2
    close(act, a, torch.bfloat16, "chain: gate/up + SwiGLU")
    assert (res.cpu() - r2).abs().max() <= 2e-2 * r2.abs().max()
    close(out, want, torch.bfloat16, "chain: last product")
