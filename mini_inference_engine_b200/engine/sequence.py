"""Per-request state (``Sequence`` of inference_engine/sequence.py:10-44).  ``num_computed`` -- the
tokens whose keys and values are in the cache -- lives in the request's ``RequestCache`` so that
pages and progress cannot drift apart."""
from __future__ import annotations

import enum
import itertools
import time

import numpy as np

from ..cache.manager import RequestCache
from ..sampling.params import SamplingParams

_ids = itertools.count()


class Status(enum.Enum):
    WAITING = 0
    RUNNING = 1
    FINISHED = 2


class Sequence:
    def __init__(self, prompt_ids, params: SamplingParams, seq_id: int | None = None):
        self.seq_id = next(_ids) if seq_id is None else seq_id
        self.token_ids = list(prompt_ids)
        self.prompt_len = len(self.token_ids)
        # the prompt once more as an array: a portion of it goes into a step's buffer as a slice, without
        # turning two thousand Python integers into numbers again at every step
        self.prompt_array = np.asarray(self.token_ids, dtype=np.int32)
        self.params = params
        self.cache = RequestCache()
        self.status = Status.WAITING
        self.num_preemptions = 0
        self.arrival_time = time.perf_counter()
        self.first_token_time: float | None = None
        self.finish_time: float | None = None
        self.pending_index = 0           # where the step in flight will leave this request's next token
        self.ended_by_eos = False        # ended by EOS while a further step was already in flight

    @property
    def num_computed(self) -> int:
        return self.cache.num_computed

    @property
    def num_tokens(self) -> int:
        return len(self.token_ids)

    @property
    def num_new_tokens(self) -> int:
        return self.num_tokens - self.cache.num_computed

    @property
    def output_ids(self) -> list:
        return self.token_ids[self.prompt_len:]

    @property
    def num_output_tokens(self) -> int:
        return self.num_tokens - self.prompt_len
