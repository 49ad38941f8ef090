"""RMS norm: x / sqrt(mean(x^2) + eps) * w, sums in 32-bit (src/math/ops.rs:1-4,
src/gpu/rmsnorm.glsl:13-26), fused with the residual add that precedes it as the
reference's unused add_rmsnorm shader does (src/gpu/add_rmsnorm.glsl:1-32)."""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from ..weights.loader import TensorRequest, WeightStore
from .base import FUSE_MAX_TOKENS, DeferredNorm, Part, StepContext, Stream
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm(Part):
    """params: size, eps.  tensors: weight [size]."""

    def tensor_requests(self) -> List[TensorRequest]:
        return [TensorRequest(self.spec.tensors["weight"], (self.p["size"],), init="ones")]

    def load(self, store: WeightStore) -> None:
        self.weight = store.get(self.tensor_requests()[0])
        self._ones = None

    graph_class = ()

    def fold_weight(self) -> torch.Tensor:
        """The weight, for a consumer that multiplies it into the columns of its own matrix."""
        return self.weight

    def apply(self, stream: Stream, ctx: StepContext, rows: Optional[torch.Tensor] = None,
              buffer: str = "normed", absorbed: bool = False):
        """Adds the stream's pending term into x and returns the normalised rows.  With
        `rows`, only those rows are produced and x is left as it is.  absorbed: the consumer has
        this norm's weight in its matrix: it is left out here, and if the stream carries a valid
        shadow nothing is computed at all (a DeferredNorm is returned)."""
        if absorbed and rows is None and stream.pending is None and stream.xb is not None and ctx.T <= FUSE_MAX_TOKENS:
            return DeferredNorm(stream.xb, stream.ssq, stream.ssq_parts, self.p["size"], self.p["eps"])
        weight = self.weight
        if absorbed:
            if self._ones is None:
                self._ones = torch.ones_like(self.weight)
            weight = self._ones
        n = stream.x.shape[0] if rows is None else rows.numel()
        out = ctx.ws.get(buffer, (n, self.p["size"]), ctx.dtype)
        kernels.add_rmsnorm(stream.x, stream.pending, weight, self.p["eps"], out, rows=rows, write_x=rows is None)
        if rows is None:
            if stream.pending is not None:
                stream.drop_shadow()              # x has changed
            stream.pending = None
        return out
