"""The model runner: the model, its cache storage, the cache manager and the batch builder in one
place, with the step function on top.  Generation (``LLMEngine``) and trace replay
(``bin/trace_run``) both drive this object; neither has a forward pass of its own.
"""
from __future__ import annotations

import numpy as np
import torch

from ..cache.manager import CacheManager, RequestCache
from ..models.decoder import DecoderModel
from .batch import BatchBuilder, BatchRow


class ModelRunner:
    def __init__(self, model: DecoderModel, num_pages: int, page_size: int, num_state_slots: int):
        self.model = model
        self.page_size = page_size
        layout = model.cache_layout
        self.cache = CacheManager(layout.groups, num_pages, page_size, num_state_slots)
        self.storage = model.allocate_cache(num_pages, page_size, num_state_slots)
        self.builder = BatchBuilder(len(layout.groups), page_size, model.rt.device, model.spec.max_position)
        self.has_state = bool(layout.state)

    # ------------------------------------------------------------------ rows
    def make_row(self, rc: RequestCache, tokens, want) -> BatchRow:
        """The batch row of a request whose pages for ``tokens`` are already reserved."""
        if self.has_state and rc.num_computed == 0 and rc.state_slot:
            self.storage.clear_state_slot(rc.state_slot)
        toks = tokens if isinstance(tokens, np.ndarray) else list(tokens)      # an array (a prompt portion) goes through as it is
        return BatchRow(toks, rc.num_computed, rc.table_arrays(), rc.state_slot, want)

    # ------------------------------------------------------------------ the step function
    @torch.inference_mode()
    def step(self, rows: list[BatchRow]) -> torch.Tensor:
        """Runs the rows as one batch from the cache and returns float32 logits
        [wanted places in row order, vocab]."""
        ctx = self.builder.build(rows)
        return self.model.step(ctx)

    def run(self, entries) -> torch.Tensor:
        """``entries``: (RequestCache, tokens, want) per request.  Reserves pages (and a state slot
        on a request's first tokens), steps, then advances every request.  Raises if pages run
        out: callers that can run out (the scheduler) reserve by themselves and call ``step``."""
        rows = []
        for rc, tokens, want in entries:
            if not self.cache.take_state_slot(rc):
                raise RuntimeError("no state slot free")
            if not self.cache.reserve(rc, len(tokens)):
                raise RuntimeError(f"cache pages ran out: a request needs {self.cache.pages_needed(rc, len(tokens))} "
                                   f"more, {[p.num_free for p in self.cache.pools]} free")
            rows.append(self.make_row(rc, tokens, want))
        logits = self.step(rows)
        for rc, tokens, _ in entries:
            self.cache.advance(rc, len(tokens))
        return logits
