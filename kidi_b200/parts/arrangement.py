"""How a layer's parts are wired around the residual stream.

`pre_norm` is the reference's Qwen3 block (src/kidi/layers/qwen3.cpp:111-122):
    h = x + mixer(input_norm(x));  out = h + feed_forward(post_norm(h))
Each sum is handed to the stream as a pending delta and formed by the next norm, in
32-bit.

Interface of an arrangement: `__init__(spec, env, parts)` with the layer's parts by
role name, `children()`, and `forward(stream, ctx, views, owns_cache)`.
"""
from __future__ import annotations

from typing import Dict

from .base import Part, ResidualStream
from .registry import register_part


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

    def forward(self, stream: ResidualStream, ctx, views, owns_cache: bool) -> None:
        stream.add(self.mixer.forward(self.input_norm.forward(stream), ctx, views, owns_cache))
        stream.add(self.feed_forward.forward(self.post_norm.forward(stream), ctx))
