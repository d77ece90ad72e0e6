"""The scheduler's decisions on the host, with a step function that only does the bookkeeping
(no GPU): admission under the token budget, portions, decodes first, finishing and freeing, what
happens when pages run out, and the same decisions as the reference's scheduler on recorded traces
(tests/golden/scheduler.json, made by tests/golden/make_golden.py)."""
import pytest

from conftest import golden
from mini_inference_engine_b200.cache import CacheManager, GroupSpec
from mini_inference_engine_b200.config import EngineConfig
from mini_inference_engine_b200.engine.scheduler import Scheduler
from mini_inference_engine_b200.engine.sequence import Sequence, Status
from mini_inference_engine_b200.sampling import SamplingParams


def make(num_blocks, budget=2048, max_num_seqs=256, chunked=True, slots=None):
    cfg = EngineConfig(max_num_batched_tokens=budget, max_num_seqs=max_num_seqs, enable_chunked_prefill=chunked)
    cache = CacheManager([GroupSpec("full")], num_blocks, 16, num_state_slots=slots or max_num_seqs)
    return Scheduler(cfg, cache), cache


def fake_step(sched, cache, batch, token=7):
    """The engine's bookkeeping after a model step (inference_engine/engine.py:212-229)."""
    for s, n in batch:
        last = s.num_computed + n == s.num_tokens
        cache.advance(s.cache, n)
        if last:
            s.token_ids.append(token)
            if s.num_output_tokens >= s.params.max_tokens:
                sched.finish(s)


def run(sched, cache, seqs, limit=5000):
    steps = []
    while sched.has_work():
        assert len(steps) < limit, "the scheduler does not terminate"
        batch = sched.schedule()
        steps.append([(seqs.index(s), n) for s, n in batch])
        fake_step(sched, cache, batch)
        cache.check()
    return steps


@pytest.mark.parametrize("name", ["roomy", "tight_pages", "tiny_budget"])
def test_same_decisions_as_the_reference_scheduler(name):
    g = golden("scheduler")[name]
    case = g["case"]
    sched, cache = make(case["num_blocks"], case["budget"], case["max_num_seqs"])
    seqs = [Sequence([1] * p, SamplingParams(max_tokens=m, ignore_eos=True))
            for p, m in zip(case["prompts"], case["max_tokens"])]
    for s in seqs:
        sched.add(s)
    steps = run(sched, cache, seqs)
    assert [[list(x) for x in st] for st in steps] == g["steps"]
    assert sched.num_preemptions == g["preemptions"]
    assert cache.num_free() == g["free_at_end"]


def test_budget_cuts_prompts_and_decodes_go_first():
    sched, cache = make(64, budget=10)
    a, b = Sequence([1] * 25, SamplingParams(max_tokens=3)), Sequence([1] * 4, SamplingParams(max_tokens=3))
    sched.add(a), sched.add(b)
    assert sched.schedule() == [(a, 10)]
    fake_step(sched, cache, [(a, 10)])
    assert sched.schedule() == [(a, 10)]
    fake_step(sched, cache, [(a, 10)])
    batch = sched.schedule()
    assert batch == [(a, 5), (b, 4)]                     # the rest of a, then b is admitted in the same step
    fake_step(sched, cache, batch)
    batch = sched.schedule()
    assert batch == [(a, 1), (b, 1)] and all(s.num_new_tokens == 1 for s, _ in batch)
    c = Sequence([1] * 30, SamplingParams(max_tokens=2))
    sched.add(c)
    fake_step(sched, cache, batch)
    assert sched.schedule() == [(a, 1), (b, 1), (c, 8)]   # decodes first, the prompt gets what is left


def test_without_chunking_a_prompt_waits_for_a_whole_budget():
    sched, cache = make(64, budget=16, chunked=False)
    a, b = Sequence([1] * 10, SamplingParams(max_tokens=2)), Sequence([1] * 10, SamplingParams(max_tokens=2))
    sched.add(a), sched.add(b)
    assert sched.schedule() == [(a, 10)]                  # b's 10 tokens do not fit the remaining 6


def test_max_num_seqs_and_head_of_line_blocking():
    sched, cache = make(6, budget=512, max_num_seqs=2)    # 5 usable pages, watermark 1
    a = Sequence([1] * 60, SamplingParams(max_tokens=2))  # 4 pages
    b = Sequence([1] * 40, SamplingParams(max_tokens=2))  # 3 pages: does not fit beside a
    c = Sequence([1] * 2, SamplingParams(max_tokens=2))   # would fit, but b is ahead of it
    for s in (a, b, c):
        sched.add(s)
    assert sched.schedule() == [(a, 60)]
    assert list(sched.waiting) == [b, c]


def test_pages_run_out_newest_request_is_preempted_and_recomputed():
    sched, cache = make(6, budget=512)                    # 5 usable pages
    a, b = Sequence([1] * 32, SamplingParams(max_tokens=40)), Sequence([1] * 32, SamplingParams(max_tokens=40))
    sched.add(a), sched.add(b)
    seqs = [a, b]
    batch = sched.schedule()
    assert batch == [(a, 32), (b, 32)]                    # 2 + 2 pages, one left
    fake_step(sched, cache, batch)
    batch = sched.schedule()                              # both need a 3rd page at position 32: only one is there
    assert batch == [(a, 1)]
    assert b.status is Status.WAITING and b.num_computed == 0 and b.cache.tables == [[]]
    assert b.num_preemptions == 1 and sched.num_preemptions == 1 and list(sched.waiting) == [b]
    assert b.num_tokens == 33                             # its generated token is kept and recomputed
    fake_step(sched, cache, batch)
    steps = run(sched, cache, seqs)
    assert a.num_output_tokens == 40 and b.num_output_tokens == 40
    assert cache.num_free() == 5
    # b came back only after a had finished and was fed prompt + its kept token in one portion
    assert (1, 33) in [x for st in steps for x in st]


def test_the_requester_itself_is_preempted_when_it_is_the_newest():
    sched, cache = make(4, budget=512)                    # 3 usable pages
    a = Sequence([1] * 16, SamplingParams(max_tokens=64))
    b = Sequence([1] * 15, SamplingParams(max_tokens=64))
    sched.add(a), sched.add(b)
    batch = sched.schedule()
    assert batch == [(a, 16), (b, 15)]
    fake_step(sched, cache, batch)
    batch = sched.schedule()                              # a takes the last page; b then needs none yet
    fake_step(sched, cache, batch)
    assert batch == [(a, 1), (b, 1)]
    batch = sched.schedule()                              # b needs a 2nd page, none left: b is the newest, b goes
    assert batch == [(a, 1)] and b.status is Status.WAITING and sched.num_preemptions == 1


def test_no_admission_in_a_step_that_preempted():
    sched, cache = make(6, budget=512)
    a, b = Sequence([1] * 32, SamplingParams(max_tokens=40)), Sequence([1] * 32, SamplingParams(max_tokens=40))
    c = Sequence([1] * 2, SamplingParams(max_tokens=2))
    sched.add(a), sched.add(b)
    fake_step(sched, cache, sched.schedule())
    sched.add(c)
    batch = sched.schedule()                              # preempts b; c (and b) must wait for the next step
    assert batch == [(a, 1)] and list(sched.waiting) == [b, c]


def test_a_request_that_can_never_fit_is_known_beforehand():
    sched, cache = make(6)                                # 5 usable pages, watermark 1 -> 64 positions
    assert sched.can_ever_fit(64) and not sched.can_ever_fit(65)


def test_finish_frees_pages_and_slot_at_once():
    sched, cache = make(16, slots=2)
    a = Sequence([1] * 20, SamplingParams(max_tokens=1))
    sched.add(a)
    batch = sched.schedule()
    assert a.cache.state_slot == 1 and cache.num_free() == 13
    fake_step(sched, cache, batch)
    assert a.status is Status.FINISHED and cache.num_free() == 15 and a.cache.state_slot == 0
    assert not sched.has_work()


def test_admission_waits_for_a_state_slot():
    sched, cache = make(32, slots=1)
    a, b = Sequence([1] * 3, SamplingParams(max_tokens=2)), Sequence([1] * 3, SamplingParams(max_tokens=2))
    sched.add(a), sched.add(b)
    assert sched.schedule() == [(a, 3)]
    assert list(sched.waiting) == [b]


@pytest.mark.parametrize("seed", range(8))
def test_random_workloads_keep_the_invariants(seed):
    """Random prompts and output lengths, arrivals spread over the run, pools from roomy to so tight
    that requests are preempted: every step keeps the budget, runs a request at most once, puts the
    decoded tokens first, covers what it runs with pages, and in the end everything ran to its length
    and every page and slot is back."""
    import random
    rng = random.Random(seed)
    budget = rng.choice([16, 40, 64, 256])
    max_seqs = rng.choice([2, 4, 8])
    chunked = seed % 4 != 3
    longest = 20 if not chunked else 90            # without chunking a prompt must fit a budget whole
    num_blocks = rng.choice([12, 16, 24, 64])
    sched, cache = make(num_blocks, budget=budget, max_num_seqs=max_seqs, chunked=chunked, slots=max_seqs)
    todo = []
    for _ in range(rng.randrange(5, 14)):
        p, o = rng.randrange(1, min(longest, budget if not chunked else longest) + 1), rng.randrange(1, 30)
        if sched.can_ever_fit(p + o):
            todo.append(Sequence(list(range(p)), SamplingParams(max_tokens=o, ignore_eos=True)))
    assert todo
    want = {id(s): (s.prompt_len, s.params.max_tokens) for s in todo}
    pending, done, steps = list(todo), [], 0
    while pending or sched.has_work():
        steps += 1
        assert steps < 20000, "the scheduler does not terminate"
        while pending and rng.random() < 0.4:
            sched.add(pending.pop(0))
        if not sched.has_work():
            sched.add(pending.pop(0))
        batch = sched.schedule()
        assert batch, "work is left but nothing was scheduled"
        assert sum(n for _, n in batch) <= budget and all(n >= 1 for _, n in batch)
        assert len({id(s) for s, _ in batch}) == len(batch)
        kinds = [s.num_new_tokens == 1 for s, _ in batch]
        assert kinds == sorted(kinds, reverse=True), "decoded tokens come first"
        assert len(sched.running) <= max_seqs
        for s, n in batch:
            assert s.status is Status.RUNNING and n <= s.num_new_tokens
            assert (chunked or n == s.num_new_tokens)
            assert all(len(t) * 16 >= s.num_computed + n for t in s.cache.tables)
            assert s.cache.state_slot != 0
        for s in sched.waiting:
            assert s.num_computed == 0 and s.cache.state_slot == 0 and s.cache.tables in ([], [[]])
        before = set(id(s) for s in sched.running)
        fake_step(sched, cache, batch)
        cache.check()
        done += [s for s, _ in batch if s.status is Status.FINISHED]
        assert before >= set(id(s) for s in sched.running)
    assert sorted(id(s) for s in done) == sorted(want)
    for s in done:
        assert (s.prompt_len, s.num_output_tokens) == want[id(s)]
    assert cache.num_free() == cache.pools[0].num_usable
    assert cache.state_pool.num_free == cache.state_pool.num_usable
