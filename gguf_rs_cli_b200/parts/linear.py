"""A dense projection y = x W^T (+ b) with W stored [out, in] as in the model folder
(src/tensor/dequant.rs:258-259).  The reference does these products with its own
kernels, not a library (src/gpu/f32_gemv.glsl, src/tensor/dequant.rs:315-317); so does
this: the tensor-core kernel where its sizes fit, the CUDA-core kernel otherwise and
everywhere in 32-bit mode.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import StepContext


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, name: str = "linear"):
        assert weight.dim() == 2
        self.weight, self.bias, self.name = weight, bias, name
        self.out_features, self.in_features = weight.shape

    def __call__(self, x: torch.Tensor, ctx: StepContext, out_dtype: Optional[torch.dtype] = None,
                 buffer: Optional[str] = None) -> torch.Tensor:
        T = x.shape[0]
        out = ctx.ws.get(buffer or self.name, (T, self.out_features), out_dtype or ctx.dtype)
        return kernels.gemm(x, self.weight, self.bias, out)
