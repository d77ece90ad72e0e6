"""Grouped-query attention over the paged cache (the mixer of Llama).

Projections q, k, v are fused into one matrix by concatenation on the output dimension, as the
reference does (inference_engine/model.py:103-107); q and k are rotated by the position part, k and
v are written to the layer's pages, and every new token attends causally to its request's
positions through the block table -- prompt portions and single decoded tokens in one kernel
(the reference has three paths: inference_engine/model.py:128-159).  ``window`` (None for Llama)
limits a query at position p to keys in (p - window, p].
"""
from __future__ import annotations

import math

import torch

from ..kernels import attention as attn_kernels
from ..weights.loader import TensorSpec
from .base import KVNeed, Mixer, build_part, register_part


class Attention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, position,
                 bias: bool = False, window: int | None = None, scale: float | None = None):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if head_dim % 16 or not 16 <= head_dim <= 256:
            raise ValueError(f"head_dim {head_dim}: the attention kernels take multiples of 16 from 16 to 256")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.bias = bias
        self.window = window
        self.scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)   # inference_engine/model.py:91
        self.position = build_part("position", position)

    def tensor_specs(self):
        H, Hkv, D, h = self.num_heads, self.num_kv_heads, self.head_dim, self.hidden_size
        specs = {"q_proj.weight": TensorSpec((H * D, h)), "k_proj.weight": TensorSpec((Hkv * D, h)),
                 "v_proj.weight": TensorSpec((Hkv * D, h)), "o_proj.weight": TensorSpec((h, H * D))}
        if self.bias:
            specs.update({"q_proj.bias": TensorSpec((H * D,), "zeros"), "k_proj.bias": TensorSpec((Hkv * D,), "zeros"),
                          "v_proj.bias": TensorSpec((Hkv * D,), "zeros")})
        specs.update(self.position.tensor_specs())       # a position encoding with tensors of its own
        return specs

    def bind(self, tensors, rt):
        self.rt = rt
        parts = [tensors[n + "_proj.weight"] for n in "qkv"]
        if len({p.dtype for p in parts}) > 1:          # mixed storage: widen to the widest
            parts = [p.float() for p in parts]
        self.w_qkv = rt.place(torch.cat(parts, 0))
        self.b_qkv = None
        if self.bias:
            self.b_qkv = rt.place(torch.cat([tensors[n + "_proj.bias"].float() for n in "qkv"], 0).to(
                torch.float32 if rt.dtype == torch.float32 else torch.bfloat16))
        self.w_o = rt.place(tensors["o_proj.weight"])
        self.position.bind({n: tensors[n] for n in self.position.tensor_specs()}, rt)

    def cache_need(self):
        return KVNeed(self.num_kv_heads, self.head_dim, self.window)

    takes_sink = True

    def kernel_sources(self):
        import torch as _torch
        names = self.rt.product_sources(self.w_qkv, self.w_o) | self.position.kernel_sources()
        if self.rt.dtype == _torch.float32 or self.head_dim > 128:
            names.add("attention_simt")
        if self.rt.dtype != _torch.float32 and self.head_dim <= 128:
            names |= {"attention_decode", "attention_prefill_tc" if self.head_dim in (64, 128) else "attention_prefill"}
        return names

    def defers_norm(self, num_tokens: int) -> bool:
        return self.rt.defers_norm(num_tokens, self.w_qkv)

    def forward(self, x, ctx, cache, sink=None):
        H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        out = self.rt.empty(ctx.num_tokens, H * D)
        if getattr(self.position, "rotates_in_attention", None) and self.position.rotates_in_attention(x, self.w_qkv, ctx, cache):
            qkv = self.rt.linear(x, self.w_qkv, self.b_qkv)
            attn_kernels.attention(qkv, ctx, cache, out, H, Hkv, D, self.scale, self.window, rope=self.position.tables())
        else:
            qkv = self.position.project_rotate_and_store(x, self.w_qkv, self.b_qkv, ctx, cache, H, Hkv)
            attn_kernels.attention(qkv, ctx, cache, out, H, Hkv, D, self.scale, self.window)
        if sink is not None:
            done = self.rt.linear_into_stream(out, self.w_o, None, sink)
            if done is not None:
                return done
        return self.rt.linear(out, self.w_o)


register_part("mixer", "attention", Attention)
