"""Token embedding (opens the float32 residual stream) and the output head
(inference_engine/model.py:96,113,168,185).  A tied head multiplies by the embedding table."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Part, register_part


class Embedding(Part):
    def __init__(self, vocab_size: int, hidden_size: int):
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size

    def tensor_specs(self):
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def bind(self, tensors, rt):
        self.rt = rt
        self.weight = rt.place(tensors["weight"])

    def kernel_sources(self):
        return {"embedding"}

    def forward(self, ctx):
        res = self.rt.empty(ctx.num_tokens, self.hidden_size, dtype=torch.float32)
        return ops.embedding(self.weight, ctx.token_ids, res, ctx.token_feedback)


class LinearHead(Part):
    """logits = x W^T in float32; ``tied`` takes W from the embedding (same tensor name)."""

    def __init__(self, vocab_size: int, hidden_size: int, tied: bool = False):
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.tied = tied

    def tensor_specs(self):
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def bind(self, tensors, rt, shared=None):
        self.rt = rt
        self.weight = shared if shared is not None else rt.place(tensors["weight"])

    def kernel_sources(self):
        return self.rt.product_sources(self.weight)

    def forward(self, x):
        return self.rt.linear(x, self.weight, None, out_dtype=torch.float32)


register_part("embedding", "embedding", Embedding)
register_part("head", "linear_head", LinearHead)
