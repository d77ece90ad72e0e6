"""SwiGLU feed-forward: down(silu(gate(x)) * up(x)).  gate and up are fused into one matrix by
concatenation on the output dimension (inference_engine/model.py:109,180-181)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import FeedForward, register_part


class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {"gate_proj.weight": TensorSpec((i, h)), "up_proj.weight": TensorSpec((i, h)),
                "down_proj.weight": TensorSpec((h, i))}

    def bind(self, tensors, rt):
        self.rt = rt
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.w_gate_up = rt.place(torch.cat([g, u], 0))
        self.w_down = rt.place(tensors["down_proj.weight"])

    def forward(self, x, ctx):
        gu = self.rt.linear(x, self.w_gate_up)
        act = self.rt.empty(x.shape[0], self.intermediate_size)
        ops.swiglu(gu, act)
        return self.rt.linear(act, self.w_down)


register_part("feed_forward", "swiglu", SwiGLU)
