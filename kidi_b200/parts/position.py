"""Position encodings.

`rotary` is the reference's table: freq_i = 1 / theta^(2i/d) for i < d/2,
angle = float(position) * freq_i, cos and sin of it, all in 32-bit, positions from
0 (src/kidi/model/qwen3.cpp:138-157). A mixer that rotates its queries and keys looks
the encoding up by name in `env.positions` and hands `cos`/`sin` to its kernel.

Interface of a position encoding: `on_embeddings(stream, ctx)` (may change the
embeddings; rotary does nothing there) and whatever its mixers agree to read from it
(`cos`, `sin`, `rotary_dim` here).
"""
from __future__ import annotations

import torch

from ..errors import invalid_argument
from .base import Part
from .registry import register_part


@register_part("position", "rotary")
class RotaryEncoding(Part):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.head_dim = int(spec.param("head_dim"))
        self.rotary_dim = int(spec.param("rotary_dim", self.head_dim))
        self.theta = float(spec.param("theta"))
        self.max_positions = int(spec.param("max_positions"))
        if self.rotary_dim <= 0 or self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise invalid_argument("the rotary width must be even and at most the head width")
        self._tables = None

    def _build(self):
        # Built at first use, on the host in 32-bit, then moved to the device once.
        if self._tables is None:
            half = self.rotary_dim // 2
            # The reference takes the power with the C library's 32-bit powf, which rounds correctly
            # in all but rare cases; a vectorised 32-bit power may be one unit off in the last
            # place, which the position multiplies (1e-4 in the cosine at position 1,000). So the
            # power is taken in 64-bit from the 32-bit base and exponent and rounded once.
            index = torch.arange(half, dtype=torch.float32)
            exponent = (2.0 * index) / torch.tensor(float(self.rotary_dim), dtype=torch.float32)
            power = torch.pow(torch.tensor(self.theta, dtype=torch.float32).double(), exponent.double()).float()
            frequency = 1.0 / power
            angle = torch.arange(self.max_positions, dtype=torch.float32)[:, None] * frequency[None, :]
            self._tables = (torch.cos(angle).contiguous().to(self.env.device),
                            torch.sin(angle).contiguous().to(self.env.device))
        return self._tables

    @property
    def cos(self) -> torch.Tensor:
        return self._build()[0]

    @property
    def sin(self) -> torch.Tensor:
        return self._build()[1]

    def on_embeddings(self, stream, ctx) -> None:
        return None
