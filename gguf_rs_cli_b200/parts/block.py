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
    graph_class = ()

    def __init__(self, mixer, feed_forward, norms):
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, norms
        self.absorbed = {"mixer": False, "feed_forward": False}

    def fuse(self) -> None:
        """After the weights are loaded: a part that can take the weight of the norm in front of it into
        its own matrix does so (then that norm costs no kernel when the stream carries a shadow)."""
        for name, part in (("mixer", self.mixer), ("feed_forward", self.feed_forward)):
            give = getattr(self.norms[name], "fold_weight", None)
            take = getattr(part, "absorb_input_norm", None)
            if give and take and not self.absorbed[name]:
                self.absorbed[name] = bool(take(give()))

    def forward(self, stream: Stream, ctx: StepContext, run: RunView) -> None:
        h = self._norm("mixer", stream, ctx)
        ctx.mark("norm")
        if getattr(self.mixer, "accepts_residual", False):
            term = self.mixer.forward(h, ctx, run, residual=stream)
        else:
            term = self.mixer.forward(h, ctx, run)
        self._add(stream, term)
        h = self._norm("feed_forward", stream, ctx)
        ctx.mark("ff_norm")
        if getattr(self.feed_forward, "accepts_residual", False):
            term = self.feed_forward.forward(h, ctx, residual=stream)
        else:
            term = self.feed_forward.forward(h, ctx)
        self._add(stream, term)

    def _norm(self, name: str, stream: Stream, ctx: StepContext):
        if self.absorbed[name]:
            return self.norms[name].apply(stream, ctx, absorbed=True)
        return self.norms[name].apply(stream, ctx)

    @staticmethod
    def _add(stream: Stream, term) -> None:
        """A part that has added its term to the stream itself returns None."""
        if term is not None:
            stream.pending = term
            stream.drop_shadow()
