"""y = x W^T for a weight stored [out, in], without bias.

This is the reference's Linear with `transpose=true, bias=false`
(src/kidi/layers/linear.cpp:98-101,181-190). It is a helper that parts own, not a
registered part. Which kernel runs follows the element types:

* a 32-bit input or a 32-bit weight: the 32-bit CUDA-core product (ascending-k fused
  multiply-adds; no reduced-precision matrix mode);
* bfloat16 by bfloat16 with few rows (decode): the weight-streaming tensor-core
  kernel of this package, when the shape fits it;
* bfloat16 by bfloat16 otherwise: the vendor matrix library through `torch.mm`, which
  is where the reference's CUDA engine calls a library too
  (docs/cuda-performance-plan.md:47-52).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops


class Linear:
    def __init__(self, weight: torch.Tensor):
        if weight.dim() != 2:
            raise ValueError("a linear weight is a matrix [out, in]")
        self.weight = weight
        self.out_features, self.in_features = weight.shape

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        out_dtype = out_dtype or x.dtype
        weight = self.weight
        if x.dtype == torch.float32 or weight.dtype == torch.float32:
            return ops.gemm_simt(x, weight, out_dtype, out=out)
        from ..kernels import skinny
        if skinny.fits(x, weight):
            return skinny.gemm(x, weight, out_dtype, out=out)
        if weight.shape[1] % 8 or x.stride(0) % 8:  # the library wants 16-byte rows; keep odd widths exact
            return ops.gemm_simt(x, weight, out_dtype, out=out)
        if out is not None:
            return torch.mm(x, weight.t(), out_dtype=out_dtype, out=out) if out_dtype != x.dtype else \
                torch.mm(x, weight.t(), out=out)
        if out_dtype != x.dtype:
            return torch.mm(x, weight.t(), out_dtype=out_dtype)
        return torch.mm(x, weight.t())
