"""Block arrangements: how norms, mixer and feed-forward sit around the residual stream."""

from __future__ import annotations

from .base import Block, ResidualStream, register_part


class PreNormResidualBlock(Block):
    """x += mixer(norm_1(x)); x += feed_forward(norm_2(x))
    (the non-parallel branch of yalis/external/model.py:414-438).
    Each addition is parked in the stream and performed by the next norm."""

    slots = {"position": "position", "norm_1": "norm", "mixer": "mixer", "norm_2": "norm",
             "feed_forward": "feed_forward"}

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        h = self.norm_1.forward(stream)
        stream.add(self.mixer.forward(h, ctx, cache))
        h = self.norm_2.forward(stream)
        stream.add(self.feed_forward.forward(h, ctx))


register_part("block", "pre_norm_residual", PreNormResidualBlock)
