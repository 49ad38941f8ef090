"""Arrangements of a layer's parts around the residual stream."""
from __future__ import annotations

from .base import RunView, StepContext, Stream
from .registry import register_block


@register_block("prenorm")
class PreNormBlock:
    """x += mixer(norm_m(x)); x += ff(norm_f(x)) (src/model/llama.rs:361-404).  The sums
    are not done here: each term is left pending on the stream and the next norm adds it
    in 32-bit while it normalises."""

    norm_names = ("mixer", "feed_forward")

    def __init__(self, mixer, feed_forward, norms):
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, norms

    def forward(self, stream: Stream, ctx: StepContext, run: RunView) -> None:
        h = self.norms["mixer"].apply(stream, ctx)
        stream.pending = self.mixer.forward(h, ctx, run)
        h = self.norms["feed_forward"].apply(stream, ctx)
        stream.pending = self.feed_forward.forward(h, ctx)
