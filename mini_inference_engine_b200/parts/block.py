"""The arrangement of parts in a layer.  ``prenorm_residual`` is Llama's: the mixer and the
feed-forward each read a normed copy of the residual stream and add their output to it.  The sum
is fused into the *next* norm, so a block takes the pending ``delta`` and returns the next one
(inference_engine/model.py:169-184: the MLP output and the residual go into the next layer's fused
add+norm, after the last layer into the final norm)."""
from __future__ import annotations

from .base import Part, ResidualSink, register_part


def _sink_for(producer, consumer, norm, res, num_tokens):
    """The offer to ``producer`` (None if it would not take one): it may add to the stream itself when
    the part behind ``norm`` can take that norm as a factor on its first product."""
    if not getattr(producer, "takes_sink", False) or consumer is None or norm is None:
        return None
    ok = getattr(consumer, "defers_norm", None)
    return ResidualSink(res, norm) if ok is not None and ok(num_tokens) else None


class Block(Part):
    """An arrangement of parts.  ``roles`` names the parts it is made of and the category each is
    built from (role -> "mixer" | "feed_forward" | "norm" | ...); the model builds them from the
    layer's description and passes them to the constructor by role name.  A block has one cache: what
    ``cache_need()`` says (by default its ``mixer``'s need, nothing for a block without one)."""
    roles: dict = {}

    def __init__(self, **parts):
        for role, part in parts.items():
            setattr(self, role, part)
        self._roles = tuple(parts)

    def parts(self) -> list:
        return [getattr(self, r) for r in self._roles]

    def cache_need(self):
        mixer = getattr(self, "mixer", None)
        return mixer.cache_need() if mixer is not None else None

    def forward(self, delta, res, ctx, cache):
        raise NotImplementedError


class PreNormResidual(Block):
    roles = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm"}

    def forward(self, delta, res, ctx, cache, next_block=None):
        """``next_block``: the block that runs after this one, if it reads the stream through a norm
        and a mixer as this one does (then the feed-forward may prepare that norm's output)."""
        n = res.shape[0]
        x = self.mixer_norm(delta, res)
        sink = _sink_for(self.mixer, self.feed_forward, self.feed_forward_norm, res, n)
        a = self.mixer.forward(x, ctx, cache, sink) if sink is not None else self.mixer.forward(x, ctx, cache)
        x = self.feed_forward_norm(a, res)
        sink = _sink_for(self.feed_forward, getattr(next_block, "mixer", None), getattr(next_block, "mixer_norm", None), res, n)
        return self.feed_forward.forward(x, ctx, sink) if sink is not None else self.feed_forward.forward(x, ctx)


register_part("block", "prenorm_residual", PreNormResidual)
