"""Sampling on the device without a host synchronisation: one kernel per step picks a token for
every row, greedy or with temperature (inference_engine/sampling.py:13-22, whose
``bool((temperatures > 0).any())`` does synchronise).  The noise of a sampled row is keyed by
(seed, request id, output position), so a request's tokens are the same whatever else is in the
batch, however its prompt was cut, and after a preemption and recompute."""
from __future__ import annotations

import torch

from ..kernels import ops


class Sampler:
    def __init__(self, device, seed: int = 0):
        self.device = torch.device(device)
        self.seed = seed

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
