"""Dense gated feed-forward: down(act(gate(h)) * up(h)) with act = SiLU
(src/model/llama.rs:399-402, src/math/ops.rs:11).  gate and up are one matrix
[2F, E] after loading, so one product reads h once."""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..weights.loader import TensorRequest, WeightStore
from typing import Optional

from .base import DeferredNorm, Part, StepContext
from .linear import Linear
from .registry import register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP(Part):
    """params: hidden_size, intermediate_size, activation ("silu").
    tensors: gate [F, E], up [F, E], down [E, F]."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        if self.p.get("activation", "silu") != "silu":
            raise ValueError(f"gated_mlp: activation {self.p['activation']!r} is not supported (silu)")

    def tensor_requests(self) -> List[TensorRequest]:
        E, F, t = self.p["hidden_size"], self.p["intermediate_size"], self.spec.tensors
        return [TensorRequest(t["gate"], (F, E)), TensorRequest(t["up"], (F, E)), TensorRequest(t["down"], (E, F))]

    def load(self, store: WeightStore) -> None:
        g, u, d = (store.get(r) for r in self.tensor_requests())
        if g.dtype != u.dtype:
            u = u.to(g.dtype)
        # where the tensor-core product can take them, gate and up are interleaved tile by tile so
        # that its epilogue applies the activation; else they are stacked and a kernel follows
        self.fused = g.dtype == torch.bfloat16 and self.p["hidden_size"] % 8 == 0 and g.is_cuda
        if self.fused:
            self.gate_up_tiles = kernels.interleave_gate_up(g, u)
        else:
            self.gate_up = Linear(torch.cat([g, u], dim=0), name="ff.gate_up")
        self.down = Linear(d, name="ff.down")

    accepts_residual = True
    graph_class = ()              # the same launches every step

    def absorb_input_norm(self, weight: torch.Tensor) -> bool:
        """Multiplies the weight of the norm in front of this part into the gate/up matrix (only
        where the tensor-core product, which can apply the norm's per-token scale, runs it)."""
        if not self.fused:
            return False
        self.gate_up_tiles = (self.gate_up_tiles.float() * weight.float()[None, :]).to(torch.bfloat16).contiguous()
        return True

    def forward(self, h, ctx: StepContext, residual=None) -> Optional[torch.Tensor]:
        F = self.p["intermediate_size"]
        act = ctx.ws.get("ff.act", (h.shape[0], F), ctx.dtype)
        norm = dict(row_ssq=h.ssq, ssq_parts=h.parts, norm_size=h.size, eps=h.eps) if isinstance(h, DeferredNorm) else {}
        rows = h.xb if norm else h
        if self.fused and kernels.gemm_tc_supported(rows, self.gate_up_tiles):
            kernels.gemm_tc(rows, self.gate_up_tiles, None, act, swiglu_features=F, **norm)
        elif self.fused:
            raise RuntimeError("gated_mlp: the activations given do not fit the fused product it was loaded for")
        else:
            kernels.swiglu(self.gate_up(h, ctx), act)
        ctx.mark("gate_up")
        term = self.down(act, ctx, residual=residual)
        ctx.mark("down")
        return term
