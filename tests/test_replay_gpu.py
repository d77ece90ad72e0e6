"""Trace replay through bin/trace_run against the plain implementation: the same requests whole,
with the last 32 tokens one by one, in portions of changing size down to two tokens, and mixed --
up to four live requests, portions of some beside decoded tokens of others, with so few pages that
they are used again -- in float32 and in bfloat16, for two tiny configurations."""
import random

import numpy as np
import pytest
import torch

import plain_llama as pl
from conftest import TINY, plain_weights
from helpers import close, first_bad_row
from replay_driver import Replay

pytestmark = pytest.mark.gpu

LENGTHS = {"tiny_a": [5, 17, 33, 64, 100, 128, 2, 49], "tiny_b": [1, 60, 37, 255, 130, 16, 97, 200],
           "tiny_c": [3, 96, 31, 50, 17, 64, 80, 9], "tiny_d": [7, 150, 64, 33, 2, 120, 48, 191]}
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def requests_for(name, seed=0):
    rng = random.Random(seed)
    vocab = TINY[name]["vocab_size"]
    return {f"r{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(LENGTHS[name])}


_oracle_cache: dict = {}


def oracle(name, folder, dtype_name, tokens):
    """Plain logits of the whole sequence; in bfloat16 mode with activations rounded where the
    engine stores them."""
    key = (name, dtype_name, tuple(tokens))
    if key not in _oracle_cache:
        cfg = pl.read_config(folder)
        W = plain_weights(folder)
        rnd = pl.round_bf16 if dtype_name == "bfloat16" else pl.identity
        _oracle_cache[key] = pl.forward(cfg, W, tokens, rnd)
    return _oracle_cache[key]


def check(name, folder, dtype_name, got: dict, reqs: dict):
    """got[id] = {position: logits row}; every position of every request must have been asked for."""
    for rid, toks in reqs.items():
        assert sorted(got[rid]) == list(range(len(toks))), f"{rid}: positions missing"
        have = torch.from_numpy(np.stack([got[rid][p] for p in range(len(toks))]))
        want = oracle(name, folder, dtype_name, toks)
        bad = first_bad_row(have, want, DTYPES[dtype_name])
        assert bad is None, (f"{name} {dtype_name} request {rid} (length {len(toks)}): first wrong position {bad} "
                             f"(page offset {bad % 16}), error "
                             f"{(have[bad] - want[bad]).abs().max():.3e} vs scale {want.abs().max():.3e}")


def collect(got, entries, logits):
    """Files the rows of one step's output under (request, position)."""
    i = 0
    for rid, pos0, want in entries:
        for w in want:
            got.setdefault(rid, {})[pos0 + w] = logits[i]
            i += 1
    assert logits is None or i == len(logits)


CASES = [(n, d) for n in ("tiny_a", "tiny_b", "tiny_c", "tiny_d") for d in ("float32", "bfloat16")]


@pytest.mark.parametrize("name,dtype_name", CASES)
def test_whole_requests(name, dtype_name, model_folders, tmp_path):
    reqs = requests_for(name)
    got: dict = {}
    with Replay(model_folders[name], dtype_name, tmp_path, 256, TINY[name]["vocab_size"]) as rp:
        for rid, toks in reqs.items():
            out = rp.step([(rid, toks, range(len(toks)))], end=[rid])
            collect(got, [(rid, 0, range(len(toks)))], out)
    check(name, model_folders[name], dtype_name, got, reqs)


@pytest.mark.parametrize("name,dtype_name", CASES)
def test_last_32_tokens_one_by_one(name, dtype_name, model_folders, tmp_path):
    reqs = requests_for(name, 1)
    got: dict = {}
    with Replay(model_folders[name], dtype_name, tmp_path, 256, TINY[name]["vocab_size"]) as rp:
        for rid, toks in reqs.items():
            head = max(0, len(toks) - 32)
            if head:
                collect(got, [(rid, 0, range(head))], rp.step([(rid, toks[:head], range(head))]))
            for p in range(head, len(toks)):
                last = p == len(toks) - 1
                collect(got, [(rid, p, [0])], rp.step([(rid, toks[p:p + 1], [0])], end=[rid] if last else []))
    check(name, model_folders[name], dtype_name, got, reqs)


@pytest.mark.parametrize("name,dtype_name", CASES)
def test_portions_of_changing_size(name, dtype_name, model_folders, tmp_path):
    reqs = requests_for(name, 2)
    sizes = [7, 2, 16, 3, 2, 5, 33, 2, 1, 14, 2, 2, 40]
    got: dict = {}
    with Replay(model_folders[name], dtype_name, tmp_path, 256, TINY[name]["vocab_size"]) as rp:
        for k, (rid, toks) in enumerate(reqs.items()):
            p, i = 0, k                                      # each request starts at another place of the cycle
            while p < len(toks):
                n = min(sizes[i % len(sizes)], len(toks) - p)
                i += 1
                out = rp.step([(rid, toks[p:p + n], range(n))], end=[rid] if p + n == len(toks) else [])
                collect(got, [(rid, p, range(n))], out)
                p += n
    check(name, model_folders[name], dtype_name, got, reqs)


@pytest.mark.parametrize("name,dtype_name", CASES)
def test_mixed_batches_with_pages_used_again(name, dtype_name, model_folders, tmp_path):
    """Up to four live requests; every step is one batch of whatever each live request feeds next:
    a portion (2..19 tokens) while it is in its 'prompt', single tokens for its last 12.  The pool
    holds 4 x (longest length rounded up to 64) positions and requests keep arriving as others end,
    so freed pages are handed to later requests."""
    rng = random.Random(7)
    vocab = TINY[name]["vocab_size"]
    lengths = LENGTHS[name] + [l // 2 + 3 for l in LENGTHS[name]]
    reqs = {f"m{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}
    longest = -(-max(lengths) // 64) * 64
    waiting = list(reqs)
    live: dict = {}
    got: dict = {}
    owners: dict = {}            # page id -> the requests that held it at some step
    with Replay(model_folders[name], dtype_name, tmp_path, 4 * longest, vocab, extra_args=("--show-pages",)) as rp:
        steps = 0
        while waiting or live:
            while waiting and len(live) < 4 and rng.random() < 0.7:
                live[waiting.pop(0)] = 0
            if not live:
                live[waiting.pop(0)] = 0
            entries, filed, ended = [], [], []
            for rid in list(live):
                if rng.random() < 0.15 and len(live) > 1:
                    continue                                  # a request may sit a step out
                toks, p = reqs[rid], live[rid]
                left = len(toks) - p
                n = 1 if left <= 12 else min(rng.choice([2, 3, 5, 8, 16, 19]), left - 12)
                want = list(range(n))
                entries.append((rid, toks[p:p + n], want))
                filed.append((rid, p, want))
                live[rid] = p + n
                if p + n == len(toks):
                    ended.append(rid)
                    del live[rid]
            if not entries:
                continue
            collect(got, filed, rp.step(entries, end=ended))
            for rid, groups in rp.pages[rp.n - 1].items():
                for page in groups[0]:
                    assert page != 0, "the scratch page was handed to a request"
                    owners.setdefault(page, set()).add(rid)
            held_now = [p for groups in rp.pages[rp.n - 1].values() for p in groups[0]]
            assert len(held_now) == len(set(held_now)), "two requests of one step hold the same page"
            steps += 1
        assert steps > 20
    # the point of the small pool: pages did go from one request to another
    assert sum(len(r) > 1 for r in owners.values()) >= 4, f"pages were not used again: {owners}"
    assert max(owners) <= 4 * longest // 16
    check(name, model_folders[name], dtype_name, got, reqs)


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_wanted_subset_and_empty_want(dtype_name, model_folders, tmp_path):
    name = "tiny_a"
    toks = requests_for(name, 3)["r4"]
    want_full = oracle(name, model_folders[name], dtype_name, toks)
    with Replay(model_folders[name], dtype_name, tmp_path, 128, TINY[name]["vocab_size"]) as rp:
        assert rp.step([("x", toks[:50], [])]) is None        # nothing wanted: no file, cache still written
        out = rp.step([("x", toks[50:], [49, 0, 7])], end=["x"])
    close(torch.from_numpy(out), want_full[[99, 50, 57]], DTYPES[dtype_name], "subset")
