"""Grouped-query attention as a mixer.

The reference's Qwen3 attention (src/kidi/layers/qwen3.cpp:13-56): one fused
projection to q, k and v heads; an optional per-head RMSNorm on q and k followed by
rotary encoding (norm before rotation, one weight vector for all heads); scores
scaled by 1/sqrt(head_dim); query head h reads key/value head h // (heads/kv_heads);
an output projection. What this part adds is the causal rule, an optional window
and the cache: key u is visible from position p when u <= p and, with a window W,
u > p - W.

Parameters (`spec.params`): hidden_size, num_heads, num_kv_heads, head_dim, qk_norm
(bool), qk_norm_eps, position (name of a rotary encoding in `env.positions`, or None),
window (tokens, or None), scale (None: 1/sqrt(head_dim)), qkv_bias and out_bias (bool,
default false: the reference's Qwen3 projections carry none, src/kidi/layers/qwen3.cpp:14-15;
its Linear has the option, src/kidi/layers/linear.cpp:181-190), score_softcap (a score s
becomes cap * tanh(s / cap); default none) and score_slopes (one number per head: head h adds
slope * (key position - query position) to its scores; default none). The last two have no
counterpart in the reference's Qwen3; they are there so that an architecture that bounds or
shifts its scores is a specification, not a change to the kernels' arguments: such layers run
on the general attention kernel in either precision.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from ..cache.sequence_cache import KVRequest
from ..errors import invalid_argument, unsupported
from ..kernels import ops
from ..kernels.attention import AttentionLauncher
from .base import Part
from .linear import Linear
from .registry import register_part
from .spec import ParamSpec


@register_part("mixer", "attention")
class Attention(Part):
    accepts_row_scaled = True     # x may lack its norm's factor: the q/k/v product applies it
    takes_sink = True             # the output product may add its result to the residual stream itself

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.param("hidden_size"))
        self.heads = int(spec.param("num_heads"))
        self.kv_heads = int(spec.param("num_kv_heads"))
        self.head_dim = int(spec.param("head_dim"))
        self.qk_norm = bool(spec.param("qk_norm", False))
        self.qkv_bias = bool(spec.param("qkv_bias", False))
        self.out_bias = bool(spec.param("out_bias", False))
        self.eps = float(spec.param("qk_norm_eps", 1e-6))
        self.window = spec.param("window", None)
        scale = spec.param("scale", None)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(float(self.head_dim))
        if self.hidden <= 0 or self.heads <= 0 or self.kv_heads <= 0 or self.heads % self.kv_heads or self.head_dim <= 0:
            raise invalid_argument("invalid attention dimensions")
        if self.head_dim > 256:
            raise unsupported(f"head_dim {self.head_dim} exceeds 256, the widest head the kernels take")
        if self.window is not None and int(self.window) <= 0:
            raise invalid_argument("an attention window must be positive")
        name = spec.param("position", None)
        self.position = env.positions[name] if name is not None else None
        if self.position is not None and self.position.head_dim != self.head_dim:
            raise invalid_argument("the rotary encoding was built for another head width")
        self.q_width = self.heads * self.head_dim
        self.kv_width = self.kv_heads * self.head_dim
        self.qkv: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.q_norm = self.k_norm = None
        # Optional: scores bounded by score_softcap * tanh(s / score_softcap); scores of head h shifted by
        # score_slopes[h] * (key position - query position) (a list with one number per head).
        self.softcap = float(spec.param("score_softcap", 0.0) or 0.0)
        slopes = spec.param("score_slopes", None)
        if slopes is not None and len(slopes) != self.heads:
            raise invalid_argument("score_slopes needs one number per attention head")
        if self.softcap < 0:
            raise invalid_argument("score_softcap must be positive")
        self.slopes = torch.tensor([float(value) for value in slopes], dtype=torch.float32, device=env.device) \
            if slopes is not None else None
        self.launcher = AttentionLauncher(heads=self.heads, kv_heads=self.kv_heads, head_dim=self.head_dim,
                                          scale=self.scale, window=self.window, softcap=self.softcap,
                                          slopes=self.slopes)

    def parameter_specs(self) -> List[ParamSpec]:
        specs = [
            ParamSpec("qkv_proj.weight", (self.q_width + 2 * self.kv_width, self.hidden), sources=(
                ("q_proj.weight", (self.q_width, self.hidden)),
                ("k_proj.weight", (self.kv_width, self.hidden)),
                ("v_proj.weight", (self.kv_width, self.hidden)))),
            ParamSpec("o_proj.weight", (self.hidden, self.q_width)),
        ]
        if self.qkv_bias:
            specs.append(ParamSpec("qkv_proj.bias", (self.q_width + 2 * self.kv_width,), sources=(
                ("q_proj.bias", (self.q_width,)), ("k_proj.bias", (self.kv_width,)), ("v_proj.bias", (self.kv_width,)))))
        if self.out_bias:
            specs.append(ParamSpec("o_proj.bias", (self.hidden,)))
        if self.qk_norm:
            specs.append(ParamSpec("q_norm.weight", (self.head_dim,), init=("one_plus_normal", 0.1)))
            specs.append(ParamSpec("k_norm.weight", (self.head_dim,), init=("one_plus_normal", 0.1)))
        return specs

    def bind(self, tensors) -> None:
        self.qkv = Linear(tensors["qkv_proj.weight"], tensors.get("qkv_proj.bias"))
        self.out = Linear(tensors["o_proj.weight"], tensors.get("o_proj.bias"))
        if self.qk_norm:
            self.q_norm, self.k_norm = tensors["q_norm.weight"], tensors["k_norm.weight"]
            if self.q_norm.dtype != self.k_norm.dtype:
                self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()

    def cache_requests(self) -> list:
        return [KVRequest(self.kv_heads, self.head_dim, int(self.window) if self.window is not None else None)]

    def launch_signature(self, rows: int, longest: int) -> tuple:
        """The choices a captured decode step of `rows` sequences of at most `longest` tokens
        freezes for this part (the form of its decode kernel)."""
        return self.launcher.launch_signature(self.env.dtype, rows, longest, self.env.device)

    def forward(self, x, ctx, views, owns_cache: bool, sink=None) -> Optional[torch.Tensor]:
        view = views[0]
        plan = ctx.plan
        qkv = self.qkv.forward(x)
        position = self.position
        rotate = dict(cos=position.cos, sin=position.sin, rotary_dim=position.rotary_dim) if position is not None \
            else dict(cos=None, sin=None, rotary_dim=0)
        common = dict(heads=self.heads, kv_heads=self.kv_heads, head_dim=self.head_dim)
        ring = view.ring_pages > 0
        # A ring that is written before attention would lose keys that the step's
        # earlier rows still need; it is written afterwards unless the step is one
        # token per sequence. A full-history cache is written first.
        store_first = owns_cache and (not ring or plan.is_decode)
        if not owns_cache and ring and not plan.is_decode:
            raise unsupported("a layer that reads another layer's windowed cache takes one token per step")
        # One token per sequence on the tensor-core path: the attention kernel takes the rows as
        # the projection left them and does norm, rotation and the cache write itself.
        fused = owns_cache and store_first and self.launcher.fuses_rotation(plan, qkv, kv_view=view, q_norm=self.q_norm,
                                                                            k_norm=self.k_norm, **rotate)
        if not fused:
            ops.rope_store(qkv, q_norm=self.q_norm, k_norm=self.k_norm, eps=self.eps, tables=ctx.tables, kv_view=view,
                           store=store_first, **rotate, **common)
        attended = torch.empty((qkv.shape[0], self.q_width), dtype=qkv.dtype, device=qkv.device)
        keys_in_step = owns_cache and not plan.is_decode
        rotation = dict(q_norm=self.q_norm, k_norm=self.k_norm, eps=self.eps, store=True, **rotate) if fused else None
        self.launcher.run(ctx, qkv, attended, kv_view=view, keys_in_step=keys_in_step, rotation=rotation,
                          step_rows_cached=store_first and not fused)
        if owns_cache and not store_first:
            ops.rope_store(qkv, q_norm=None, k_norm=None, eps=self.eps, tables=ctx.tables, kv_view=view, store=True,
                           transform=False, cos=None, sin=None, rotary_dim=0, **common)
        return self.out.forward(attended, sink=sink)
