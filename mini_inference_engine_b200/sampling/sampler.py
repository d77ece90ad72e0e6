"""Sampling on the device without a host synchronisation: one kernel per step picks a token for
every row, greedy or with temperature (inference_engine/sampling.py:13-22, whose
``bool((temperatures > 0).any())`` does synchronise).  The noise of a sampled row is keyed by
(seed, request id, output position), so a request's tokens are the same whatever else is in the
batch, however its prompt was cut, and after a preemption and recompute."""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops


class Sampler:
    """Owns what sampling needs of a step: the per-row inputs that ride in the step's one host-to-device
    transfer (``inputs``), the rule for seeds (a request's own seed, else the engine's) and the launch."""

    def __init__(self, device, seed: int = 0):
        self.device = torch.device(device)
        self.seed = seed

    @staticmethod
    def inputs(rows: int, requests=(), turn: int = 0) -> dict:
        """The sampling inputs of a step as small host arrays, padded to ``rows`` rows (a captured step has
        its bucket's rows): temperature, request id and output position of every request that samples, and
        which row of the pinned token buffer the step fills.  ``requests`` have ``params.temperature``,
        ``seq_id``, ``token_ids`` and ``prompt_len``."""
        t = np.zeros(rows, dtype=np.float32)
        r = np.zeros(rows, dtype=np.int64)
        p = np.zeros(rows, dtype=np.int32)
        k = len(requests)
        if k:
            t[:k] = [s.params.temperature for s in requests]
            r[:k] = [s.seq_id for s in requests]
            p[:k] = [len(s.token_ids) - s.prompt_len for s in requests]
        return {"temperature": t, "request": r, "out_position": p, "host_turn": np.array([turn], dtype=np.int32)}

    def seeds_of(self, requests) -> tuple:
        """Every request's seed, and the set of seeds that matter (those of requests that draw with noise):
        one seed at most means one launch serves all rows."""
        seeds = [self.seed if s.params.seed is None else s.params.seed for s in requests]
        return seeds, {sd for sd, s in zip(seeds, requests) if s.params.temperature > 0}

    def sample_step(self, logits: torch.Tensor, extras: dict, out: torch.Tensor, seeds: list, noisy: set,
                    host_out: torch.Tensor | None = None) -> bool:
        """Samples every row of ``logits`` into ``out``.  With one seed among the noisy rows that is one
        launch, which also writes the tokens into ``host_out`` (True is returned); requests with different
        seeds of their own take one launch a row, and the caller copies the tokens to the host (False)."""
        if len(noisy) <= 1:
            self.sample(logits, extras["temperature"], extras["request"], extras["out_position"], out=out,
                        seed=next(iter(noisy)) if noisy else None, host_out=host_out, host_turn=extras["host_turn"])
            return True
        for i, sd in enumerate(seeds):
            self.sample(logits[i:i + 1], extras["temperature"][i:i + 1], extras["request"][i:i + 1],
                        extras["out_position"][i:i + 1], out=out[i:i + 1], seed=sd)
        return False

    def sample(self, logits: torch.Tensor, temperature: torch.Tensor, request: torch.Tensor,
               position: torch.Tensor, out: torch.Tensor | None = None, seed: int | None = None,
               host_out: torch.Tensor | None = None, host_turn: torch.Tensor | None = None) -> torch.Tensor:
        """logits float32 [rows, vocab]; temperature float32 [rows]; request int64 [rows];
        position int32 [rows] (index of the token being drawn among the request's outputs).
        ``host_out`` / ``host_turn``: see ``ops.sample``."""
        if out is None:
            out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        return ops.sample(logits, temperature, request, position, self.seed if seed is None else seed, out,
                          host_out, host_turn)
