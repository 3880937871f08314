"""Token embedding and the output head.

Embedding: a row gather times a scalar scale into the 32-bit residual stream
(src/kidi/layers/gemma4.cpp:68-163; scale 1 for Qwen3, src/kidi/model/qwen3.cpp:78).
Head: logits = x W^T in 32-bit at the rows that were asked for; W may be the embedding
table itself (tied). The reference's Qwen3 has no head; the generic causal path's
"final norm -> lm_head -> 32-bit logits, selected rows only" is the precedent
(src/kidi/model/gemma4.cpp:769-778,1057).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import ops
from .base import Part
from .linear import Linear
from .registry import register_part
from .spec import ParamSpec


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab = int(spec.param("vocab_size"))
        self.hidden = int(spec.param("hidden_size"))
        self.scale = float(spec.param("scale", 1.0))
        self.weight: Optional[torch.Tensor] = None

    def parameter_specs(self) -> List[ParamSpec]:
        return [ParamSpec("weight", (self.vocab, self.hidden))]

    def bind(self, tensors) -> None:
        self.weight = tensors["weight"]

    def forward(self, tokens: torch.Tensor, ctx) -> torch.Tensor:
        return ops.embedding(tokens, self.weight, self.scale)


@register_part("head", "linear_head")
class LinearHead(Part):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab = int(spec.param("vocab_size"))
        self.hidden = int(spec.param("hidden_size"))
        self.tied_to = spec.param("tied_to", None)
        self.linear: Optional[Linear] = None

    def parameter_specs(self) -> List[ParamSpec]:
        return [ParamSpec("weight", (self.vocab, self.hidden), alias_of=self.tied_to)]

    def bind(self, tensors) -> None:
        self.linear = Linear(tensors["weight"])

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        return self.linear.forward(x, out_dtype=torch.float32)
