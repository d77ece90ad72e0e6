"""Which requests run in the next step, and with how many tokens each.

The *decisions* are those of the reference's scheduler (inference_engine/scheduler.py:22-107), pinned
by recorded traces of it in the tests; the code is organised around this package's cache manager,
which holds a request's pages, state slot and progress in one ``RequestCache``.

A step's batch is drawn up as a ``_Draft`` under the token budget ``max_num_batched_tokens``:

  * requests that are decoding come first and get their one token each;
  * then requests that are part-way through their prompt get as much of the rest as the budget
    still allows (all of it or nothing when chunked prefill is off);
  * then, unless room had to be made in this very step, requests are taken from the front of the
    waiting queue while the budget, ``max_num_seqs``, the pages (less a reserve, ``watermark``) and
    the state slots allow; the queue is strictly first come first served: when its head does not
    fit, nobody behind it is tried.

Making room: when a running request cannot get the pages for its tokens, the request admitted last
loses everything it holds and goes back to the *front* of the queue with its progress at zero; the
tokens it has generated stay and are recomputed with its prompt.  This repeats until the pages
suffice or the request asking for them was itself the last one.  A request that lost its pages after
it had been put on the draft is taken off it again.

Decided here, absent from the reference: a request that can never fit (more positions than
``max_model_len`` or than the usable pages hold) is refused when it is added -- ``can_ever_fit`` --
instead of being admitted, pushed out and admitted again for ever.
"""
from __future__ import annotations

from collections import deque

from ..cache.manager import CacheManager
from ..config.engine_config import EngineConfig
from .sequence import Sequence, Status


class _Draft:
    """The batch of one step while it is being drawn up."""

    def __init__(self, budget: int):
        self.budget = budget
        self.single = []          # (request, 1): decoded tokens
        self.portions = []        # (request, n): prompt portions, running requests before new ones
        self.made_room = False    # a request was pushed out while drafting

    def put(self, seq: Sequence, n: int, decoding: bool) -> None:
        (self.single if decoding else self.portions).append((seq, n))
        self.budget -= n

    def still_running(self) -> None:
        """Takes off the draft whoever was pushed out after being put on it."""
        self.single = [(s, n) for s, n in self.single if s.status is Status.RUNNING]
        self.portions = [(s, n) for s, n in self.portions if s.status is Status.RUNNING]

    def rows(self) -> list:
        return self.single + self.portions


class Scheduler:
    def __init__(self, cfg: EngineConfig, cache: CacheManager):
        self.cfg = cfg
        self.cache = cache
        self.waiting: deque = deque()
        self.running: list = []          # in order of admission: the last one is the first to be pushed out
        self.num_preemptions = 0
        # pages an admission must leave free (a hundredth of the pool, at least one): room for the
        # running requests' next pages (inference_engine/scheduler.py:29-30)
        self.watermark = max(1, min(p.num_pages for p in cache.pools) // 100)

    # ------------------------------------------------------------------ the queue
    def can_ever_fit(self, num_positions: int) -> bool:
        need = self.cache.max_pages_for(num_positions)
        return all(n + self.watermark <= pool.num_usable for n, pool in zip(need, self.cache.pools))

    def add(self, seq: Sequence) -> None:
        self.waiting.append(seq)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ making room
    def _push_out(self, seq: Sequence) -> None:
        """Recompute preemption: nothing of the request's cache survives, its tokens do."""
        self.running.remove(seq)
        self.cache.free(seq.cache)                 # pages and state slot back, progress to zero
        seq.status = Status.WAITING
        seq.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(seq)               # ahead of everyone who has not started yet

    def _pages_for(self, seq: Sequence, n: int, draft: _Draft) -> bool:
        """Pages for the next ``n`` tokens of a running request, at the cost of the requests
        admitted after it if need be.  False when ``seq`` itself was the one to go."""
        while not self.cache.reserve(seq.cache, n):
            last_in = self.running[-1]
            self._push_out(last_in)
            draft.made_room = True
            if last_in is seq:
                return False
        return True

    # ------------------------------------------------------------------ one step's batch
    def schedule(self) -> list:
        draft = _Draft(self.cfg.max_num_batched_tokens)
        whole_prompts_only = not self.cfg.enable_chunked_prefill

        mid_prompt = []
        for seq in tuple(self.running):            # a copy: making room shortens the list
            if seq.status is not Status.RUNNING:
                continue                           # pushed out a moment ago
            if len(seq.token_ids) - seq.cache.num_computed != 1:
                mid_prompt.append(seq)
            elif draft.budget == 0:
                break
            elif self._pages_for(seq, 1, draft):
                draft.put(seq, 1, decoding=True)

        for seq in mid_prompt:
            rest = seq.num_new_tokens
            if seq.status is not Status.RUNNING or rest <= 1 or draft.budget == 0:
                continue
            n = min(rest, draft.budget)
            if whole_prompts_only and n < rest:
                continue
            if self._pages_for(seq, n, draft):
                draft.put(seq, n, decoding=False)

        draft.still_running()
        if not draft.made_room:
            self._admit(draft, whole_prompts_only)
        return draft.rows()

    def _admit(self, draft: _Draft, whole_prompts_only: bool) -> None:
        while self.waiting and draft.budget > 0 and len(self.running) < self.cfg.max_num_seqs:
            seq = self.waiting[0]
            n = min(seq.num_new_tokens, draft.budget)
            if whole_prompts_only and n < seq.num_new_tokens:
                return
            if not self.cache.can_reserve(seq.cache, n, watermark=self.watermark):
                return
            if not self.cache.take_state_slot(seq.cache):
                return
            self.cache.reserve(seq.cache, n, watermark=self.watermark)
            self.waiting.popleft()
            seq.status = Status.RUNNING
            self.running.append(seq)
            draft.put(seq, n, decoding=False)

    def finish(self, seq: Sequence) -> None:
        """Ends a request wherever it is: running (what it holds goes back) or waiting again after
        having been pushed out (it holds nothing)."""
        if seq.status is Status.RUNNING:
            self.running.remove(seq)
            self.cache.free(seq.cache)
        elif seq.status is Status.WAITING and seq in self.waiting:
            self.waiting.remove(seq)
        seq.status = Status.FINISHED
