"""y = x W^T (+ b) for a weight stored [out, in] and an optional bias [out].

This is the reference's Linear with `transpose=true` and its optional bias
(src/kidi/layers/linear.cpp:98-101,181-190). It is a helper that parts own, not a
registered part. The bias is kept in 32-bit and added in the epilogue of this package's
product kernels (after the vendor library's product, by a kernel of its own). Which
kernel runs follows the element types:

* a 32-bit input or a 32-bit weight: the 32-bit CUDA-core product (ascending-k fused
  multiply-adds; no reduced-precision matrix mode);
* bfloat16 by bfloat16 with up to 8 rows (decode): the weight-streaming `mma.sync`
  kernel of this package (`kernels/skinny.py`);
* bfloat16 by bfloat16 with 9 to 16 rows and a large weight (16384 output features or
  more: the fused gate/up projection, the output head): this package's tcgen05 kernel
  (`kernels/tcgen05.py`: TMA-fed, accumulating in tensor memory), which streams such
  weights as fast as the vendor library does up to there (and takes up to 64 rows when
  KIDI_B200_TCGEN05_MAX_ROWS says so);
* bfloat16 by bfloat16 with 1,024 rows or more (prompts): the tcgen05 kernel again, in its
  compute-bound form (whole tiles of 128 features x 256 tokens, a persistent block per SM);
* bfloat16 by bfloat16 otherwise (17 to 1,023 rows): the vendor matrix library through
  `torch.mm`, which is where the reference's CUDA engine calls a library too
  (docs/cuda-performance-plan.md:47-52).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import RowScaled


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        if weight.dim() != 2:
            raise ValueError("a linear weight is a matrix [out, in]")
        self.weight = weight
        self.out_features, self.in_features = weight.shape
        if bias is not None and bias.shape != (self.out_features,):
            raise ValueError("a linear bias has one element per output feature")
        self.bias = bias.float().contiguous() if bias is not None else None

    def forward(self, x, out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None,
                sink=None) -> Optional[torch.Tensor]:
        """`x`: a matrix or a `RowScaled` (rows that lack their norm's factor: the weight-streaming
        kernel applies it to its result, any other kernel gets plain rows). `sink`: a
        `ResidualSink`; if the weight-streaming kernel runs and the sink's norm takes prepared
        rows, the result goes into the residual stream and None is returned."""
        from ..kernels import skinny
        weight, bias = self.weight, self.bias
        factors = None
        if isinstance(x, RowScaled):
            if skinny.supports(x.values, weight) and x.values.shape[0] <= skinny.MAX_ROWS:
                x, factors = x.values, x.factors
            else:
                x = x.plain()
        out_dtype = out_dtype or x.dtype
        if sink is not None and out is None and out_dtype == x.dtype and skinny.supports(x, weight) \
                and x.shape[0] <= skinny.MAX_ROWS:
            norm_weight = sink.norm.prepared_weight() if hasattr(sink.norm, "prepared_weight") else None
            stream = sink.stream
            if norm_weight is not None and stream.pending is None and stream.hidden.shape == (x.shape[0], weight.shape[0]):
                values, parts = skinny.gemm_into_residual(x, weight, stream.hidden, norm_weight, bias=bias,
                                                          factors=factors)
                stream.prepared = (sink.norm, values, parts)
                return None
        if factors is not None:
            return skinny.gemm(x, weight, out_dtype, out=out, bias=bias, factors=factors)
        if x.dtype == torch.float32 or weight.dtype == torch.float32:
            return ops.gemm_simt(x, weight, out_dtype, out=out, bias=bias)
        from ..kernels import tcgen05
        if skinny.fits(x, weight):
            return skinny.gemm(x, weight, out_dtype, out=out, bias=bias)
        if (weight.shape[0] >= tcgen05.MIN_FEATURES and tcgen05.fits(x, weight)) or tcgen05.fits_prompt(x, weight):
            return tcgen05.gemm(x, weight, out_dtype, out=out, bias=bias)
        if weight.shape[1] % 8 or x.stride(0) % 8:  # the library wants 16-byte rows; keep odd widths exact
            return ops.gemm_simt(x, weight, out_dtype, out=out, bias=bias)
        ops.note("library_mm")
        if out is not None:
            result = torch.mm(x, weight.t(), out_dtype=out_dtype, out=out) if out_dtype != x.dtype else \
                torch.mm(x, weight.t(), out=out)
        elif out_dtype != x.dtype:
            result = torch.mm(x, weight.t(), out_dtype=out_dtype)
        else:
            result = torch.mm(x, weight.t())
        return ops.add_bias(result, bias) if bias is not None else result
