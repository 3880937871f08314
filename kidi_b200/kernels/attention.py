"""Chooses the attention kernel for a step.

The generic kernel takes every element type, head width up to 256 and any number of
heads, for prompts and for single tokens, and is the only one the 32-bit engine uses.
The bfloat16 engine uses the tensor-core kernels where the shape fits them.
"""
from __future__ import annotations

from . import ops


def run(ctx, qkv, out, *, heads, kv_heads, head_dim, scale, window, kv_view, keys_in_step) -> None:
    ops.attention_generic(qkv, out, heads=heads, kv_heads=kv_heads, head_dim=head_dim, scale=scale, window=window,
                          tables=ctx.tables, kv_view=kv_view, keys_in_step=keys_in_step)
