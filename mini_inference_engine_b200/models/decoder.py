"""The generic decoder: a model is what its ``ModelSpec`` says -- an embedding, layers put together
from registered parts, a run order, a final norm and a head.  Nothing here names an architecture.

``step(ctx)`` is the one step function: it runs exactly the tokens of the batch (prompt portions
beside single decoded tokens), reading earlier positions from the cache and writing the new
ones, and returns float32 logits at the wanted positions only
(the reference's ``LlamaModel.forward``, inference_engine/model.py:161-185, returns every row in a
pure-decode step; here the wanted positions are always explicit).
"""
from __future__ import annotations

import inspect

import torch

from ..cache.storage import CacheLayout, CacheStorage
from ..config.model_config import ModelSpec
from ..parts.base import Runtime, StepContext, build_part, part_class
from ..weights.loader import TensorSpec, check_and_bind


def _layer_parts(layer_spec):
    """Builds the parts a layer's block class asks for (its ``roles``: role name -> part category)
    from the layer's description and hands them to the block by role name."""
    cls = part_class("block", layer_spec.block)
    roles = cls.roles
    if set(roles) != set(layer_spec.parts):
        raise ValueError(f"block {layer_spec.block!r} is made of {', '.join(sorted(roles))}; the layer describes "
                         f"{', '.join(sorted(layer_spec.parts))}")
    built = {role: build_part(roles[role], layer_spec.parts[role]) for role in roles}
    return cls(**built), [(layer_spec.parts[role].prefix, built[role]) for role in roles]


class _Skeleton:
    """The parts of a model, built but not yet given weights."""

    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = build_part("embedding", spec.embedding)
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = build_part("head", spec.head)
        self.blocks = []
        self.named = [(spec.embedding.prefix, self.embedding), (spec.final_norm.prefix, self.final_norm)]
        if spec.head.prefix != spec.embedding.prefix:
            self.named.append((spec.head.prefix, self.head))
        for ls in spec.layers:
            block, named = _layer_parts(ls)
            self.blocks.append(block)
            self.named.extend(named)
        for e in spec.run_order:
            if not 0 <= e.layer < len(self.blocks):
                raise ValueError(f"run order names layer {e.layer}; the model has {len(self.blocks)}")

    def expected(self) -> dict[str, TensorSpec]:
        out: dict[str, TensorSpec] = {}
        for prefix, part in self.named:
            for local, ts in part.tensor_specs().items():
                name = prefix + local
                if name in out and tuple(out[name].shape) != tuple(ts.shape):
                    raise ValueError(f"two parts want {name} with different shapes")
                out[name] = ts
        return out


def expected_tensors(spec: ModelSpec) -> dict[str, TensorSpec]:
    """Every checkpoint tensor the model of ``spec`` reads, by full name."""
    return _Skeleton(spec).expected()


class DecoderModel:
    def __init__(self, spec: ModelSpec, state: dict, rt: Runtime, where: str = "checkpoint"):
        sk = _Skeleton(spec)
        self.spec = spec
        self.rt = rt
        tied = spec.head.prefix == spec.embedding.prefix
        tensors = check_and_bind(state, sk.expected(), ignore=tuple(spec.ignore), where=where)
        for prefix, part in sk.named:
            local = {n: tensors[prefix + n] for n in part.tensor_specs()}
            part.bind(local, rt)
        if tied:
            sk.head.bind({}, rt, shared=sk.embedding.weight)
        self.embedding, self.final_norm, self.head, self.blocks = sk.embedding, sk.final_norm, sk.head, sk.blocks
        if rt.device.type == "cuda":
            # what this model launches is known now: compile what is still missing side by side
            from ..kernels import build
            names = set()
            for _, part in sk.named:
                names |= part.kernel_sources()
            build.prepare(names)
        self.run_order = spec.run_order
        # a block that can be told which block runs after it (to prepare that block's first norm)
        self._takes_next = ["next_block" in inspect.signature(b.forward).parameters for b in self.blocks]
        needs: dict = {}
        for e in self.run_order:                   # a cache's shape is what the layers that use it declare
            need = self.blocks[e.layer].cache_need()
            if e.cache in needs and needs[e.cache] != need:
                raise ValueError(f"cache {e.cache} is used by layers with different needs: {needs[e.cache]} and {need}")
            needs[e.cache] = need
        first_writer = {}
        for e in self.run_order:
            if e.writes_cache:
                first_writer.setdefault(e.cache, e.layer)
            elif e.cache not in first_writer:
                raise ValueError(f"layer {e.layer} reads cache {e.cache} before any entry has written it")
        self.cache_layout = CacheLayout.from_needs(needs)
        self.storage: CacheStorage | None = None
        self._caches: list = []

    # ------------------------------------------------------------------ cache
    def allocate_cache(self, num_pages, page_size: int, num_state_slots: int) -> CacheStorage:
        self.storage = CacheStorage(self.cache_layout, num_pages, page_size, num_state_slots, self.rt.dtype,
                                    self.rt.device)
        self._caches = [self.storage.layer_cache(e.cache, e.writes_cache) for e in self.run_order]
        return self.storage

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for obj in [self.embedding, self.final_norm, self.head] + [p for b in self.blocks for p in b.parts()]:
            for v in vars(obj).values():
                if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
        return total

    # ------------------------------------------------------------------ the step function
    def step(self, ctx: StepContext) -> torch.Tensor:
        if self.storage is None:
            raise RuntimeError("allocate_cache() must be called before step()")
        with self.rt.step_scope():
            return self._step(ctx)

    def _step(self, ctx: StepContext) -> torch.Tensor:
        res = self.embedding.forward(ctx)
        delta = None
        last = len(self.run_order) - 1
        for i, (entry, cache) in enumerate(zip(self.run_order, self._caches)):
            block = self.blocks[entry.layer]
            if self._takes_next[entry.layer] and i < last:
                delta = block.forward(delta, res, ctx, cache, next_block=self.blocks[self.run_order[i + 1].layer])
            else:
                delta = block.forward(delta, res, ctx, cache)
        if ctx.want.numel() == 0:
            return torch.empty(0, self.spec.vocab_size, dtype=torch.float32, device=self.rt.device)
        x = self.final_norm(delta, res, rows=ctx.want)
        return self.head.forward(x)
