"""The arrangement of parts in a layer.  ``prenorm_residual`` is Llama's: the mixer and the
feed-forward each read a normed copy of the residual stream and add their output to it.  The sum
is fused into the *next* norm, so a block takes the pending ``delta`` and returns the next one
(inference_engine/model.py:169-184: the MLP output and the residual go into the next layer's fused
add+norm, after the last layer into the final norm)."""
from __future__ import annotations

from .base import Part, build_part, register_part


class PreNormResidual(Part):
    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm

    def forward(self, delta, res, ctx, cache):
        x = self.mixer_norm(delta, res)
        a = self.mixer.forward(x, ctx, cache)
        x = self.feed_forward_norm(a, res)
        return self.feed_forward.forward(x, ctx)


register_part("block", "prenorm_residual", PreNormResidual)
