"""Interfaces of the parts a layer is put together from, and the registries that map a
``PartSpec.kind`` to a class.

A part knows its own sizes and constants (constructor parameters) and nothing about the model it
sits in: tensor names are relative to a prefix that the model's description supplies, and what a
part needs of the past (pages of keys and values, a window of them, a fixed-size state, nothing)
is declared through ``cache_need()`` so that the cache manager can group layers by need.

Interfaces (duck-typed; the base classes below only document them and hold the defaults):

  every part      tensor_specs() -> {local tensor name: TensorSpec}
                  bind(tensors: {local name: device tensor}, rt: Runtime) -> None
  norm            __call__(delta | None, res, out_rows=None) -> x      res += delta; x = norm(res)
  mixer           cache_need() -> KVNeed | StateNeed | None
                  forward(x[T, hidden], ctx: StepContext, cache: LayerCache) -> [T, hidden]
  feed-forward    forward(x[T, hidden], ctx) -> [T, hidden]
  position        rotate_and_store(qkv, ctx, cache, heads, kv_heads)   rotate q (in place) and k, write k, v to the cache
                  project_rotate_and_store(x, w_qkv, b_qkv, ctx, cache, heads, kv_heads) -> qkv   (may fuse the three)
  block           forward(delta, res, ctx, cache) -> delta'            (arrangement of the above)
  embedding       forward(ctx) -> res [T, hidden] float32
  head            forward(x[W, hidden]) -> logits [W, vocab] float32

The reference has none of this: its one model reads its constants from the configuration inside
its methods (inference_engine/model.py:84-115,161-185).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..config.model_config import PartSpec
from ..weights.loader import TensorSpec

CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")
_REGISTRY: dict[str, dict[str, type]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str, cls: type) -> None:
    if category not in _REGISTRY:
        raise KeyError(f"unknown part category {category!r}; one of {', '.join(CATEGORIES)}")
    _REGISTRY[category][kind] = cls


def part_class(category: str, kind: str) -> type:
    try:
        return _REGISTRY[category][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY.get(category, {})))
        raise KeyError(f"no {category} part registered as {kind!r} (registered: {known})") from None


def build_part(category: str, spec: PartSpec):
    return part_class(category, spec.kind)(**spec.params)


# --------------------------------------------------------------------------- what a layer needs of the past

@dataclass(frozen=True)
class KVNeed:
    """Pages of keys and values: all positions (``window`` None) or the last ``window``."""
    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size state per request: a tensor of ``shape`` and ``dtype`` per state slot,
    zeroed when a request takes the slot."""
    shape: tuple
    dtype: torch.dtype = torch.float32


@dataclass
class LayerCache:
    """What the model hands a mixer: its layer's storage and where to find the batch's view of it."""
    group: int = -1                 # index into ctx.block_tables / ctx.slots for page-backed layers
    k: torch.Tensor | None = None   # [pages, kv_heads, page_size, head_dim]
    v: torch.Tensor | None = None
    page_size: int = 0
    state: torch.Tensor | None = None   # [slots + 1, *shape]; slot 0 is scratch
    writes: bool = True             # False when this run of the layer only reads another layer's cache


# --------------------------------------------------------------------------- what a step gives every part

@dataclass
class StepContext:
    """One step's batch on the device.  Row r is one request with ``row_q_len[r]`` new tokens at
    flat offsets ``row_q_start[r]``..; after the step its cache holds ``row_ctx_len[r]`` positions.
    ``host`` mirrors the per-row numbers as Python lists for parts that plan on the host."""
    num_tokens: int
    num_rows: int
    token_ids: torch.Tensor            # int32 [T]
    positions: torch.Tensor            # int32 [T]
    token_row: torch.Tensor            # int32 [T]
    row_q_start: torch.Tensor          # int32 [R]
    row_q_len: torch.Tensor            # int32 [R]
    row_ctx_len: torch.Tensor          # int32 [R]
    state_slots: torch.Tensor          # int32 [R]
    block_tables: list                 # per cache group: int32 [R, max_pages]
    slots: list                        # per cache group: int32 [T] flat cache slot of each new token
    want: torch.Tensor                 # int32 [W] flat token indices whose logits are wanted
    max_q_len: int = 1
    max_ctx_len: int = 1
    host: dict = field(default_factory=dict)
    extras: dict = field(default_factory=dict)   # small per-step device arrays that rode along (sampling inputs)
    token_feedback: torch.Tensor | None = None   # int32: tokens the previous step sampled; a token id -(k+1) means entry k


@dataclass
class ResidualSink:
    """What a block may offer a mixer or feed-forward in place of adding its output afterwards: the
    float32 stream ``res`` and the norm that reads the stream next.  A part that takes the offer adds
    its output to ``res`` itself (in its last product's epilogue) and returns a StreamUpdated."""
    res: torch.Tensor
    norm: object


@dataclass
class StreamUpdated:
    """Returned instead of an output: the stream already holds the sum.  ``deferred`` is what the part
    prepared for ``norm`` (see kernels/gemm_tc.py: DeferredNorm), or None."""
    norm: object
    deferred: object


class Runtime:
    """Device, activation type and the matrix product for that type.  ``float32`` runs every
    product on CUDA cores in true 32-bit; ``bfloat16`` uses the tensor-core product for 16-bit
    weights and the CUDA-core one for a matrix that the checkpoint holds in 32 bits."""

    def __init__(self, device, dtype: torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype must be torch.float32 or torch.bfloat16, got {dtype}")
        self.device = torch.device(device)
        self.dtype = dtype

    def place(self, t: torch.Tensor) -> torch.Tensor:
        """A checkpoint tensor on the device in its compute type: everything float32 in the
        32-bit mode; in bfloat16 mode 16-bit tensors stay bfloat16 and 32-bit ones stay 32-bit."""
        if t.dtype.is_floating_point:
            if self.dtype == torch.float32:
                t = t.to(torch.float32)
            elif t.dtype != torch.float32:
                t = t.to(torch.bfloat16)
        return t.to(self.device).contiguous()

    def empty(self, *shape, dtype=None) -> torch.Tensor:
        return torch.empty(*shape, dtype=dtype or self.dtype, device=self.device)

    def linear(self, x, w: torch.Tensor, bias=None, out_dtype=None) -> torch.Tensor:
        from ..kernels import linear as _linear
        return _linear.linear(x, w, bias, out_dtype or self.dtype)

    def product_sources(self, *weights) -> set:
        """The kernel sources behind ``linear`` for these weights."""
        if self.dtype == torch.float32 or any(w is not None and w.dtype == torch.float32 for w in weights):
            return {"gemm_simt"} if self.dtype == torch.float32 else {"gemm_simt"} | self._tc_sources()
        return self._tc_sources()

    @staticmethod
    def _tc_sources() -> set:
        from ..kernels import gemm_tc
        return {"gemm_tcgen05", "gemm_pair_tc"} | ({"gemm_chain"} if gemm_tc.chain_enabled else set())

    def step_scope(self):
        """A context for one step of a model: in bfloat16 the fused few-token products queued inside it go
        out as chains, one launch for several products (kernels/gemm_tc.py: chaining)."""
        if self.dtype == torch.bfloat16:
            from ..kernels import gemm_tc
            return gemm_tc.chaining()
        import contextlib
        return contextlib.nullcontext()

    def defers_norm(self, num_tokens: int, w: torch.Tensor) -> bool:
        """Whether the product with ``w`` can take the norm in front of it as a factor on its sums
        (its input then comes as a DeferredNorm from ``linear_into_stream``)."""
        from ..kernels import linear as _linear
        return self.dtype == torch.bfloat16 and _linear.splits_k_on_tcgen05(num_tokens, w)

    def linear_into_stream(self, x, w: torch.Tensor, bias, sink: ResidualSink):
        """The last product of a part, adding to the stream of ``sink`` in its epilogue and preparing
        the input of the product behind ``sink.norm``.  Returns a StreamUpdated, or None where that
        is not possible (the part then returns its output as usual)."""
        from ..kernels import linear as _linear
        args = getattr(sink.norm, "deferred_args", None)
        if args is None or self.dtype != torch.bfloat16:
            return None
        weight, eps = args()
        d = _linear.linear_into_stream(x, w, bias, sink.res, weight, eps)
        return None if d is False else StreamUpdated(sink.norm, d)


class Part:
    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {}

    def kernel_sources(self) -> set:
        """Names of the kernel sources (csrc/<name>.cu) this part launches once bound; the model
        compiles the ones still missing side by side when it is built."""
        return set()

    def bind(self, tensors: dict, rt: Runtime) -> None:
        self.rt = rt


class Mixer(Part):
    def cache_need(self):
        return None

    def forward(self, x, ctx: StepContext, cache: LayerCache):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, ctx: StepContext):
        raise NotImplementedError
