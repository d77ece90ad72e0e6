"""Continuous batching with chunked prefill and recompute preemption: the decisions of
``Scheduler`` in inference_engine/scheduler.py:22-107, over this package's cache manager.

Every step a fresh batch is built under the token budget ``max_num_batched_tokens``:
  1. every running request that is decoding gets its one token (growth ignores the watermark);
  2. running requests that are part-way through their prompt get their next portion;
  3. waiting requests are admitted in arrival order, their prompts cut to the remaining budget;
     an admission must leave ``watermark`` pages free and takes a state slot; if the head of the
     queue does not fit, nothing behind it is admitted; nothing is admitted in a step that had to
     preempt.
When pages run out for a running request, the most recently admitted request is preempted: all it
holds is given back, its progress is reset to zero (its generated tokens are kept and recomputed
with the prompt) and it goes to the *front* of the waiting queue.  If the request that needs the
pages is itself the most recent one, it is the one preempted.

Decided here and absent from the reference: a request that can never fit -- more positions than
``max_model_len`` or than all usable pages hold -- is refused when it is added (``can_ever_fit``),
instead of being admitted, preempted and re-admitted for ever.
"""
from __future__ import annotations

from collections import deque

from ..cache.manager import CacheManager
from ..config.engine_config import EngineConfig
from .sequence import Sequence, Status


class Scheduler:
    def __init__(self, cfg: EngineConfig, cache: CacheManager):
        self.cfg = cfg
        self.cache = cache
        self.waiting: deque = deque()
        self.running: list = []
        self.num_preemptions = 0
        # keep about 1% of the pages free when admitting, so running requests can grow
        self.watermark = max(1, min(p.num_pages for p in cache.pools) // 100)

    # ------------------------------------------------------------------ queue
    def can_ever_fit(self, num_positions: int) -> bool:
        need = self.cache.max_pages_for(num_positions)
        return all(n + self.watermark <= pool.num_usable for n, pool in zip(need, self.cache.pools))

    def add(self, seq: Sequence) -> None:
        self.waiting.append(seq)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ preemption
    def _preempt(self, seq: Sequence) -> None:
        self.running.remove(seq)
        self.cache.free(seq.cache)            # pages, state slot, num_computed = 0
        seq.status = Status.WAITING
        seq.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(seq)

    def _reserve_or_preempt(self, seq: Sequence, n: int) -> bool:
        """Pages for ``seq``'s next n tokens, evicting the newest running requests if needed.
        False if ``seq`` itself had to go."""
        while not self.cache.reserve(seq.cache, n):
            victim = self.running[-1]
            self._preempt(victim)
            if victim is seq:
                return False
        return True

    # ------------------------------------------------------------------ one step's batch
    def schedule(self) -> list:
        budget = self.cfg.max_num_batched_tokens
        decodes, prefills = [], []
        preemptions_before = self.num_preemptions

        in_prompt = []
        for seq in list(self.running):                                   # 1. decodes
            if seq.status is not Status.RUNNING:
                continue
            if len(seq.token_ids) - seq.cache.num_computed != 1:
                in_prompt.append(seq)
                continue
            if budget == 0:
                break
            if self._reserve_or_preempt(seq, 1):
                decodes.append((seq, 1))
                budget -= 1

        for seq in in_prompt:                                            # 2. prompts in flight
            if seq.status is not Status.RUNNING or seq.num_new_tokens <= 1 or budget == 0:
                continue
            n = min(seq.num_new_tokens, budget)
            if not self.cfg.enable_chunked_prefill and n < seq.num_new_tokens:
                continue
            if self._reserve_or_preempt(seq, n):
                prefills.append((seq, n))
                budget -= n

        # a request scheduled above may have been evicted to make room for a later one
        decodes = [(s, n) for s, n in decodes if s.status is Status.RUNNING]
        prefills = [(s, n) for s, n in prefills if s.status is Status.RUNNING]

        preempted_now = self.num_preemptions != preemptions_before         # 3. admissions
        while self.waiting and budget > 0 and len(self.running) < self.cfg.max_num_seqs and not preempted_now:
            seq = self.waiting[0]
            n = min(seq.num_new_tokens, budget)
            if not self.cfg.enable_chunked_prefill and n < seq.num_new_tokens:
                break
            if not self.cache.can_reserve(seq.cache, n, watermark=self.watermark):
                break
            if not self.cache.take_state_slot(seq.cache):
                break
            self.cache.reserve(seq.cache, n, watermark=self.watermark)
            self.waiting.popleft()
            seq.status = Status.RUNNING
            self.running.append(seq)
            prefills.append((seq, n))
            budget -= n

        return decodes + prefills

    def finish(self, seq: Sequence) -> None:
        """Ends a request wherever it is: running (its pages and slot go back) or waiting again after
        a preemption (it holds nothing)."""
        if seq.status is Status.RUNNING:
            self.running.remove(seq)
            self.cache.free(seq.cache)
        elif seq.status is Status.WAITING and seq in self.waiting:
            self.waiting.remove(seq)
        seq.status = Status.FINISHED
