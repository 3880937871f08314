"""How a layer's parts are wired around the residual stream.

`pre_norm` is the reference's Qwen3 block (src/kidi/layers/qwen3.cpp:111-122):
    h = x + mixer(input_norm(x));  out = h + feed_forward(post_norm(h))
Each sum is handed to the stream as a pending delta and formed by the next norm, in
32-bit.

Interface of an arrangement: `__init__(spec, env, parts)` with the layer's parts by
role name, `children()`, and `forward(stream, ctx, views, owns_cache)`. Optionally
`first_norm()` (the norm it applies to the stream first) and, with the class attribute
`supports_next_norm`, `forward(..., next_norm=...)`: the norm that reads the stream after
this layer, so that the layer's last product can prepare the rows for it.

Norms between two products need no launch of their own when both products run on the
weight-streaming kernel (`ResidualSink`, `RowScaled` in parts/base.py): the product before
the norm adds its result to the stream and prepares the rows, the product after applies
each row's factor. The arrangement only makes the offers; parts that do not know them
get and return plain matrices.
"""
from __future__ import annotations

from typing import Dict

from .base import Part, ResidualSink, ResidualStream, plain_rows
from .registry import register_part


import os

# Which norms are folded into the products around them: "all", "post" (the norm after the mixer only),
# "none".
FOLD_NORMS = os.environ.get("KIDI_B200_FOLD_NORMS", "all")


def normed_for(norm: Part, stream: ResidualStream, consumer: Part):
    """The stream's rows normalised by `norm`, as a `RowScaled` where `consumer` takes one."""
    if getattr(consumer, "accepts_row_scaled", False) and hasattr(norm, "prepared_weight"):
        return norm.forward(stream, scaled=True)
    return plain_rows(norm.forward(stream))


def sink_for(part: Part, stream: ResidualStream, norm):
    """The offer to `part` to add its result to the stream itself, for `norm` to find prepared."""
    if norm is not None and FOLD_NORMS != "none" and getattr(part, "takes_sink", False) and hasattr(norm, "prepared_weight"):
        return {"sink": ResidualSink(stream, norm)}
    return {}


@register_part("arrangement", "pre_norm")
class PreNormBlock(Part):
    ROLES = {"input_norm": "norm", "mixer": "mixer", "post_norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self, spec, env, parts: Dict[str, Part]):
        super().__init__(spec, env)
        self.input_norm = parts["input_norm"]
        self.mixer = parts["mixer"]
        self.post_norm = parts["post_norm"]
        self.feed_forward = parts["feed_forward"]

    def children(self):
        return (self.input_norm, self.mixer, self.post_norm, self.feed_forward)

    def cache_requests(self) -> list:
        return self.mixer.cache_requests()

    supports_next_norm = True

    def first_norm(self) -> Part:
        return self.input_norm

    def forward(self, stream: ResidualStream, ctx, views, owns_cache: bool, next_norm=None) -> None:
        stream.add(self.mixer.forward(normed_for(self.input_norm, stream, self.mixer), ctx, views, owns_cache,
                                      **sink_for(self.mixer, stream, self.post_norm)))
        stream.add(self.feed_forward.forward(normed_for(self.post_norm, stream, self.feed_forward), ctx,
                                             **sink_for(self.feed_forward, stream, next_norm if FOLD_NORMS == "all" else None)))
