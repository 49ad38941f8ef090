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
from .base import FUSE_MAX_TOKENS, DeferredNorm, StepContext, Stream


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, name: str = "linear"):
        assert weight.dim() == 2
        self.weight, self.bias, self.name = weight, bias, name
        self.out_features, self.in_features = weight.shape

    def tensor_core(self) -> bool:
        """Whether the tensor-core product takes this matrix (bfloat16, rows of a multiple of 8)."""
        w = self.weight
        return w.dtype == torch.bfloat16 and w.is_cuda and w.shape[1] % 8 == 0 and w.stride(0) % 8 == 0

    def fold_input_scale(self, scale: torch.Tensor) -> None:
        """W[:, k] *= scale[k]: the weight of the norm in front of this projection, multiplied in."""
        self.weight = (self.weight.float() * scale.float()[None, :]).to(self.weight.dtype).contiguous()

    def __call__(self, x, ctx: StepContext, out_dtype: Optional[torch.dtype] = None, buffer: Optional[str] = None,
                 residual: Optional[Stream] = None) -> Optional[torch.Tensor]:
        """x: rows [T, in], or a DeferredNorm (then the product applies the norm's scale).  With
        `residual`, and where the tensor-core product can do it, the result is added to the stream in
        the product's epilogue (x += result, shadow left for the next norm) and None is returned."""
        T = x.shape[0]
        norm = dict(row_ssq=x.ssq, ssq_parts=x.parts, norm_size=x.size, eps=x.eps) if isinstance(x, DeferredNorm) else {}
        rows = x.xb if norm else x
        if residual is not None and T <= FUSE_MAX_TOKENS and self.tensor_core() \
                and kernels.gemm_tc_supported(rows, self.weight) and residual.x.shape == (T, self.out_features):
            xb = ctx.ws.get("stream.xb", residual.x.shape, torch.bfloat16)
            parts = (self.out_features + 127) // 128
            ssq = ctx.ws.get("stream.ssq", (parts, T), torch.float32)
            kernels.gemm_tc(rows, self.weight, self.bias, None, resid_x=residual.x, resid_xb=xb, ssq_out=ssq, **norm)
            residual.pending, residual.xb, residual.ssq, residual.ssq_parts = None, xb, ssq, parts
            return None
        out = ctx.ws.get(buffer or self.name, (T, self.out_features), out_dtype or ctx.dtype)
        if norm:
            return kernels.gemm_tc(rows, self.weight, self.bias, out, **norm)
        return kernels.gemm(x, self.weight, self.bias, out)
