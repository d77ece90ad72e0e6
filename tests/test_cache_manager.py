"""The cache manager on the host: no page is lost, held twice or freed twice, under random orders of
requests; windows give pages back; state slots; the batch packing (no GPU)."""
import random

import numpy as np
import pytest

from mini_inference_engine_b200.cache import CacheManager, GroupSpec, PageError, PagePool, RequestCache, RELEASED
from mini_inference_engine_b200.engine.batch import BatchBuilder, BatchRow


def test_pool_fifo_and_scratch_page():
    p = PagePool(6)
    assert p.num_free == 5 and p.num_usable == 5
    a = p.take(2)
    assert a == [1, 2]                                   # page 0 is never handed out
    b = p.take(3)
    assert not p.can_take(1)
    p.give_back(a)
    assert p.take(2) == [1, 2]                           # first in, first out
    p.give_back(b)
    p.check()


def test_pool_refuses_double_free_and_foreign_pages():
    p = PagePool(4)
    a = p.take(1)
    p.give_back(a)
    with pytest.raises(PageError, match="freed twice"):
        p.give_back(a)
    with pytest.raises(PageError):
        p.give_back([0])
    with pytest.raises(PageError):
        p.give_back([9])
    with pytest.raises(PageError):
        p.take(99)


def test_reserve_grows_tables_and_free_returns_everything():
    m = CacheManager([GroupSpec("full")], 10, 16, num_state_slots=2)
    rc = RequestCache()
    assert m.take_state_slot(rc) and rc.state_slot == 1
    assert m.reserve(rc, 17) and rc.tables == [[1, 2]]
    m.advance(rc, 17)
    assert m.pages_needed(rc, 15) == [0] and m.pages_needed(rc, 16) == [1]
    assert m.reserve(rc, 16)
    m.advance(rc, 16)
    assert rc.num_computed == 33 and len(rc.tables[0]) == 3
    m.free(rc)
    assert m.num_free() == 9 and rc.tables == [[]] and rc.state_slot == 0 and rc.num_computed == 0
    m.check()


def test_watermark_only_applies_when_asked():
    m = CacheManager([GroupSpec("full")], 5, 16)        # 4 usable
    a, b = RequestCache(), RequestCache()
    assert m.reserve(a, 48)                               # 3 pages
    assert not m.reserve(b, 16, watermark=1)              # an admission must leave one page free
    assert b.tables in ([], [[]])
    assert m.reserve(a, 16 + 0)                           # nothing more needed yet
    m.advance(a, 48)
    assert m.reserve(a, 1)                                # growth ignores the watermark
    assert not m.reserve(b, 1)
    m.check()


def test_reserve_is_all_or_nothing_across_groups():
    m = CacheManager([GroupSpec("full"), GroupSpec("window32", 32)], [10, 3], 16)
    rc = RequestCache()
    assert not m.reserve(rc, 48)                          # the window group has only 2 usable pages
    assert m.num_free(0) == 9 and m.num_free(1) == 2
    assert m.reserve(rc, 32)
    m.check()


def test_window_gives_pages_back_as_it_passes():
    m = CacheManager([GroupSpec("full"), GroupSpec("w", 20)], 12, 16)
    rc = RequestCache()
    total = 0
    for n in (16, 16, 7, 9, 1, 1, 30):
        assert m.reserve(rc, n)
        released = m.advance(rc, n)
        total += n
        assert released[0] == []
        # the next query at position `total` reads keys > total - 20
        first_needed = max(0, total - 20 + 1) // 16
        assert all(p == RELEASED for p in rc.tables[1][:first_needed])
        assert all(p != RELEASED for p in rc.tables[1][first_needed:])
        assert len(rc.tables[1]) == len(rc.tables[0]) == -(-total // 16)
    held = [p for p in rc.tables[1] if p != RELEASED]
    assert m.pools[1].num_free == 11 - len(held) and len(held) <= 3
    m.free(rc)
    m.check()
    assert m.pools[0].num_free == 11 and m.pools[1].num_free == 11


@pytest.mark.parametrize("seed", range(6))
def test_random_requests_never_lose_or_share_a_page(seed):
    rng = random.Random(seed)
    groups = [GroupSpec("full")] + ([GroupSpec("w", rng.choice([8, 24, 40]))] if seed % 2 else [])
    m = CacheManager(groups, 24, 16, num_state_slots=4)
    live: list = []
    for _ in range(600):
        op = rng.random()
        if op < 0.35 and len(live) < 4:
            rc = RequestCache()
            if m.take_state_slot(rc):
                live.append(rc)
        elif op < 0.85 and live:
            rc = rng.choice(live)
            n = rng.choice([1, 1, 1, 2, 5, 16, 17, 40])
            if m.reserve(rc, n, watermark=rng.choice([0, 1])):
                m.advance(rc, n)
        elif live:
            rc = live.pop(rng.randrange(len(live)))
            m.free(rc)
        m.check()
        for g in range(len(groups)):                      # no page is in two tables
            held = [p for rc in live for p in (rc.tables[g] if rc.tables else []) if p != RELEASED]
            assert len(held) == len(set(held)) and 0 not in held
            assert sorted(held) == m.pools[g].held_pages()
        slots = [rc.state_slot for rc in live]
        assert len(slots) == len(set(slots)) and 0 not in slots
        for rc in live:                                   # the arrays the batch builder gets are never stale
            if rc.tables:
                assert [t.tolist() for t in rc.table_arrays()] == rc.tables
    for rc in live:
        m.free(rc)
    m.check()
    assert all(p.num_free == p.num_usable for p in m.pools)


def test_batch_packing_positions_slots_and_wanted_places():
    b = BatchBuilder(1, 16, "cpu", max_position=128)
    rows = [BatchRow([5], 33, [[7, 2, 9]], state_slot=1, want=[0]),          # a decoded token at position 33
            BatchRow([1, 2, 3, 4, 5], 14, [[4, 6]], state_slot=2, want=[1, 4]),  # a portion crossing a page edge
            BatchRow([9, 9], 0, [[3]], state_slot=3, want=[])]
    ctx = b.build(rows)
    assert ctx.num_tokens == 8 and ctx.num_rows == 3
    assert ctx.token_ids.tolist() == [5, 1, 2, 3, 4, 5, 9, 9]
    assert ctx.positions.tolist() == [33, 14, 15, 16, 17, 18, 0, 1]
    assert ctx.token_row.tolist() == [0, 1, 1, 1, 1, 1, 2, 2]
    assert ctx.row_q_start.tolist() == [0, 1, 6] and ctx.row_q_len.tolist() == [1, 5, 2]
    assert ctx.row_ctx_len.tolist() == [34, 19, 2]
    assert ctx.slots[0].tolist() == [9 * 16 + 1, 4 * 16 + 14, 4 * 16 + 15, 6 * 16, 6 * 16 + 1, 6 * 16 + 2, 48, 49]
    assert ctx.want.tolist() == [0, 2, 5]
    assert ctx.block_tables[0].tolist() == [[7, 2, 9], [4, 6, 0], [3, 0, 0]]
    assert ctx.state_slots.tolist() == [1, 2, 3]
    assert ctx.max_q_len == 5 and ctx.max_ctx_len == 34


@pytest.mark.parametrize("seed", range(8))
def test_batch_packing_of_random_batches_token_by_token(seed):
    """Single decoded tokens beside portions, tables as lists or arrays, one or two groups, padded or
    not: every token's position, row and cache slot against the definition, one token at a time."""
    rng = random.Random(seed)
    G, ps = rng.choice([1, 2]), rng.choice([4, 16])
    b = BatchBuilder(G, ps, "cpu", max_position=4096)
    R = rng.randrange(1, 12)
    only_decode = seed % 3 == 0
    rows = []
    for _ in range(R):
        n = 1 if only_decode or rng.random() < 0.5 else rng.randrange(2, 50)
        pos0 = rng.randrange(0, 300)
        pages = -(-(pos0 + n) // ps) + rng.randrange(0, 2)
        tabs = [[rng.randrange(1, 900) for _ in range(pages)] for _ in range(G)]
        if rng.random() < 0.5:
            tabs = [np.array(t, dtype=np.int32) for t in tabs]
        toks = [rng.randrange(-4, 1000) for _ in range(n)]
        if n > 1 and rng.random() < 0.5:
            toks = np.array(toks, dtype=np.int32)
        rows.append(BatchRow(toks, pos0, tabs, rng.randrange(0, 5), sorted(rng.sample(range(n), rng.randrange(0, min(n, 3) + 1)))))
    pad = R + rng.randrange(0, 4) if seed % 2 else None
    width = max(len(t) for r in rows for t in r.tables) + rng.randrange(0, 3) if seed % 2 else None
    ctx = b.to_device(*b.pack(rows, pad_rows=pad, table_width=width))
    tok, pos, trow, want = [], [], [], []
    slots = [[] for _ in range(G)]
    for i, r in enumerate(rows):
        for j, t in enumerate(list(r.tokens)):
            if j in r.want:
                want.append(len(tok))
            tok.append(int(t)); pos.append(r.pos0 + j); trow.append(i)
            for g in range(G):
                slots[g].append(int(r.tables[g][(r.pos0 + j) // ps]) * ps + (r.pos0 + j) % ps)
    for i in range(R, pad or R):                           # scratch rows: token 0 at position 0 of page 0
        want.append(len(tok))
        tok.append(0); pos.append(0); trow.append(i)
        for g in range(G):
            slots[g].append(0)
    assert ctx.token_ids.tolist() == tok and ctx.positions.tolist() == pos and ctx.token_row.tolist() == trow
    assert ctx.want.tolist() == want
    for g in range(G):
        assert ctx.slots[g].tolist() == slots[g]
        for i, r in enumerate(rows):
            have = ctx.block_tables[g][i].tolist()
            assert have[:len(r.tables[g])] == list(map(int, r.tables[g])) and not any(have[len(r.tables[g]):])
    assert ctx.row_q_len.tolist() == [len(r.tokens) for r in rows] + [1] * ((pad or R) - R)
    assert ctx.row_ctx_len.tolist() == [r.pos0 + len(r.tokens) for r in rows] + [1] * ((pad or R) - R)
    assert ctx.state_slots.tolist() == [r.state_slot for r in rows] + [0] * ((pad or R) - R)


def test_batch_packing_padding_rows_and_extras():
    b = BatchBuilder(2, 16, "cpu")
    rows = [BatchRow([4], 20, [[3, 5], [0, 2]], 1, [0])]
    ex = {"temperature": np.array([0.5, 0, 0, 0], dtype=np.float32), "request": np.array([2 ** 40, 0, 0, 0], dtype=np.int64)}
    buf, layout = b.pack(rows, pad_rows=4, table_width=6, extras=ex)
    ctx = b.to_device(buf, layout)
    assert ctx.num_rows == 4 and ctx.num_tokens == 4 and ctx.want.tolist() == [0, 1, 2, 3]
    assert ctx.row_ctx_len.tolist() == [21, 1, 1, 1] and ctx.positions.tolist() == [20, 0, 0, 0]
    assert ctx.slots[0].tolist() == [5 * 16 + 4, 0, 0, 0] and ctx.slots[1].tolist() == [2 * 16 + 4, 0, 0, 0]
    assert ctx.block_tables[1].shape == (4, 6)
    assert ctx.extras["temperature"].tolist() == [0.5, 0, 0, 0] and ctx.extras["request"][0].item() == 2 ** 40
    assert ctx.host["real_rows"] == 1


def test_batch_packing_refuses_bad_rows():
    b = BatchBuilder(1, 16, "cpu", max_position=32)
    with pytest.raises(ValueError, match="no page"):
        b.build([BatchRow([1, 2], 15, [[3]], 0, [])])
    with pytest.raises(ValueError, match="outside"):
        b.build([BatchRow([1, 2], 0, [[3]], 0, [2])])
    with pytest.raises(ValueError, match="max_position"):
        b.build([BatchRow([1] * 3, 30, [[3, 4, 5]], 0, [])])
    with pytest.raises(ValueError, match="at least one token"):
        b.build([BatchRow([], 0, [[3]], 0, [])])
