"""RMSNorm: y = x * (1 / sqrt(mean(x^2) + eps)) * w.

The reference's RmsNorm (src/kidi/layers/gemma4.cpp:23-67; op contract
src/kidi/ops/context.cpp:1043-1082; arithmetic
src/kidi/runtime/mps/eager_kernels.metal:65-87). The norm is also where the residual
stream takes its pending delta: sum and normalisation run in one kernel, in 32-bit.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import ops
from .base import Part, ResidualStream, RowScaled
from .registry import register_part
from .spec import ParamSpec


@register_part("norm", "rms_norm")
class RMSNorm(Part):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = int(spec.param("size"))
        self.eps = float(spec.param("eps"))
        self.weight: Optional[torch.Tensor] = None

    def parameter_specs(self) -> List[ParamSpec]:
        return [ParamSpec("weight", (self.size,), init=("one_plus_normal", 0.1))]

    def bind(self, tensors) -> None:
        self.weight = tensors["weight"]

    def prepared_weight(self) -> Optional[torch.Tensor]:
        """The weight vector a product needs to prepare rows for this norm (`ResidualSink`), or
        None when this norm does not take prepared rows."""
        return self.weight if self.env.dtype == torch.bfloat16 else None

    def forward(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None, scaled: bool = False):
        """Adds the stream's pending delta and returns the normalised rows in the
        engine dtype. With `rows` (int32 indices) only those rows are produced and the
        stream itself is left untouched. With `scaled` the caller takes a `RowScaled` too:
        when the product before has prepared the rows (added its result to the stream, multiplied
        by this norm's weight, summed the squares) there is nothing left to launch."""
        prepared = stream.take_prepared(self) if rows is None else None
        if prepared is not None:
            ready = RowScaled(prepared[0], prepared[1], self.size, self.eps)
            return ready if scaled else ready.plain()
        return ops.add_rmsnorm(stream.hidden, stream.take_pending(), self.weight, self.eps, self.env.dtype,
                               row_index=rows)
