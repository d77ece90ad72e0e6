"""SwiGLU feed-forward: down(silu(gate(x)) * up(x)).  gate and up are fused into one matrix
(inference_engine/model.py:109,180-181 concatenates them on the output dimension).  In bfloat16 the
fused matrix interleaves them instead -- row 2i = gate_i, row 2i+1 = up_i -- so that the tensor-core
product can apply SwiGLU in its epilogue while both values of a pair sit side by side."""
from __future__ import annotations

import torch

from ..kernels import linear as linear_kernels
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
        self.interleaved = rt.dtype == torch.bfloat16 and g.dtype != torch.float32
        if self.interleaved:
            self.w_gate_up = rt.place(torch.stack((g, u), 1).reshape(2 * self.intermediate_size, self.hidden_size))
        else:
            self.w_gate_up = rt.place(torch.cat([g, u], 0))
        self.w_down = rt.place(tensors["down_proj.weight"])

    takes_sink = True

    def kernel_sources(self):
        return {"activation"} | self.rt.product_sources(self.w_gate_up, self.w_down)

    def defers_norm(self, num_tokens: int) -> bool:
        return self.rt.defers_norm(num_tokens, self.w_gate_up)

    def forward(self, x, ctx, sink=None):
        if self.interleaved:
            act = linear_kernels.linear_swiglu(x, self.w_gate_up, self.rt.dtype)
        else:
            gu = self.rt.linear(x, self.w_gate_up)
            act = self.rt.empty(x.shape[0], self.intermediate_size)
            ops.swiglu(gu, act)
        if sink is not None:
            done = self.rt.linear_into_stream(act, self.w_down, None, sink)
            if done is not None:
                return done
        return self.rt.linear(act, self.w_down)


register_part("feed_forward", "swiglu", SwiGLU)
