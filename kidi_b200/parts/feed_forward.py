"""Gated feed-forward: y = (act(x Wg^T) * (x Wu^T)) Wd^T.

The reference's GatedFeedForward (src/kidi/layers/gemma4.cpp:164-225): one fused
projection to [gate | up] (gate = first I columns), the activation on the gate times
up, then the down projection; no biases. SiLU is g / (1 + exp(-g))
(src/kidi/runtime/mps/eager_kernels.metal:129-137).

Parameters: hidden_size, intermediate_size, activation ("silu").
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..errors import unsupported
from ..kernels import ops
from .base import Part, RowScaled
from .linear import Linear
from .registry import register_part
from .spec import ParamSpec


@register_part("feed_forward", "gated_mlp")
class GatedFeedForward(Part):
    accepts_row_scaled = True     # x may lack its norm's factor: the gate/up product applies it
    takes_sink = True             # the down product may add its result to the residual stream itself

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.param("hidden_size"))
        self.inter = int(spec.param("intermediate_size"))
        activation = spec.param("activation", "silu")
        if activation != "silu":
            raise unsupported(f"gated feed-forward activation '{activation}' is not built (silu is)")
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def parameter_specs(self) -> List[ParamSpec]:
        return [
            ParamSpec("gate_up_proj.weight", (2 * self.inter, self.hidden), sources=(
                ("gate_proj.weight", (self.inter, self.hidden)),
                ("up_proj.weight", (self.inter, self.hidden)))),
            ParamSpec("down_proj.weight", (self.hidden, self.inter)),
        ]

    def bind(self, tensors) -> None:
        self.gate_up = Linear(tensors["gate_up_proj.weight"])
        self.down = Linear(tensors["down_proj.weight"])

    def forward(self, x, ctx, sink=None) -> Optional[torch.Tensor]:
        from ..kernels import skinny, tcgen05
        factors = None
        if isinstance(x, RowScaled):
            if skinny.supports(x.values, self.gate_up.weight) and x.values.shape[0] <= skinny.MAX_ROWS:
                x, factors = x.values, x.factors
            else:
                x = x.plain()
        if factors is not None or skinny.fits(x, self.gate_up.weight):
            gated = skinny.gemm_silu_gate(x, self.gate_up.weight, factors=factors)
        elif tcgen05.MIN_GATED_ROWS <= x.shape[0] <= tcgen05.MAX_GATED_ROWS and tcgen05.fits(x, self.gate_up.weight):
            gated = tcgen05.gemm_silu_gate(x, self.gate_up.weight)
        else:
            gated = ops.silu_gate(self.gate_up.forward(x))
        return self.down.forward(gated, sink=sink)
