"""Token embedding (a row gather, src/model/llama.rs:349) and the output head
(logits = W h, src/model/llama.rs:406-407), which falls back to the embedding table
when the folder has no matrix of its own (src/model/llama.rs:124)."""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..weights.loader import TensorRequest, WeightStore
from .base import FUSE_MAX_TOKENS, Part, StepContext, Stream
from .linear import Linear
from .registry import register_embedding, register_head


@register_embedding("embedding")
class Embedding(Part):
    """params: vocab_size, hidden_size.  tensors: weight [V, E]."""

    def tensor_requests(self) -> List[TensorRequest]:
        return [TensorRequest(self.spec.tensors["weight"], (self.p["vocab_size"], self.p["hidden_size"]))]

    graph_class = ()

    def load(self, store: WeightStore) -> None:
        self.weight = store.get(self.tensor_requests()[0])

    def forward(self, tokens: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        x = ctx.ws.get("x", (tokens.numel(), self.p["hidden_size"]), torch.float32)
        return kernels.embed(self.weight, tokens, x)

    def forward_stream(self, tokens: torch.Tensor, ctx: StepContext) -> Stream:
        """The residual stream of a step; in bfloat16 mode with the shadow (bfloat16 copy and sums of
        squares per token) that lets the first norm be deferred into the product after it."""
        if ctx.dtype != torch.bfloat16 or tokens.numel() > FUSE_MAX_TOKENS:
            return Stream(self.forward(tokens, ctx))
        T, E = tokens.numel(), self.p["hidden_size"]
        stream = Stream(ctx.ws.get("x", (T, E), torch.float32))
        stream.xb = ctx.ws.get("stream.xb", (T, E), torch.bfloat16)
        stream.ssq = ctx.ws.get("stream.ssq", ((E + 127) // 128, T), torch.float32)
        stream.ssq_parts = 1
        kernels.embed_shadow(self.weight, tokens, stream.x, stream.xb, stream.ssq)
        return stream


@register_head("lm_head")
class LMHead(Part):
    """params: vocab_size, hidden_size, tied_to (the tensor that stands in when the folder has no
    head matrix of its own, or None), tied (the configuration says the head is the embedding: the
    random-weights mode then writes no matrix for it).
    tensors: weight [V, E].  As in the reference, presence decides: a folder that has the matrix
    uses it, one that lacks it uses `tied_to` (src/model/llama.rs:124)."""

    def tensor_requests(self) -> List[TensorRequest]:
        shape = (self.p["vocab_size"], self.p["hidden_size"])
        init = None if self.p.get("tied") else "normal"
        if self.p.get("tied_to"):
            return [TensorRequest(self.spec.tensors["weight"], shape, optional=True, fallback=self.p["tied_to"], init=init)]
        return [TensorRequest(self.spec.tensors["weight"], shape, init=init)]

    graph_class = ()

    def load(self, store: WeightStore) -> None:
        self.proj = Linear(store.get(self.tensor_requests()[0]), name="logits")

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return self.proj(h, ctx, out_dtype=torch.float32)
