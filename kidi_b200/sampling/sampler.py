"""Token selection: greedy, and temperature sampling with a seed.

Greedy is the reference's only way of sampling text (argmax, ties to the lowest index,
invalid rows rejected: ARCHITECTURE.md:612-616, src/kidi/inference/decoder.cpp:72-80;
its temperature and seed options exist for speech synthesis only, src/kidi/cli/main.cpp:898-899).
Temperature sampling is this library's own: p = softmax(logits / T) in 32-bit and the
inverse of the cumulative distribution at a uniform number keyed by (seed, sequence
key, step), so that a sequence's draw does not depend on what else is in its batch. In the
32-bit engine the logits do not either (every kernel adds in an order that depends on the
position only), so a sequence generates the same tokens in any batch; the bfloat16 engine
chooses its product and attention kernels by the number of rows of a step, each of which
rounds in its own order, so there the same holds up to that rounding (a token may differ
where two logits lie closer together than it).
Both run on the device (`kernels/ops.py`: argmax, sample).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..errors import invalid_argument
from ..kernels import ops


class Sampler:
    def __init__(self, seed: int = 0):
        self.seed = int(seed)

    def select(self, logits: torch.Tensor, temperature: Optional[torch.Tensor] = None,
               keys: Optional[torch.Tensor] = None, steps: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One token id per row of `logits` (int32, on the device; -1 for a row without
        a valid score). Without `temperature` every row is greedy."""
        if temperature is None:
            return ops.argmax(logits, out=out)
        if keys is None or steps is None:
            raise invalid_argument("temperature sampling needs a key and a step per row")
        return ops.sample(logits, temperature, self.seed, keys, steps, out=out)

    def select_host(self, logits: torch.Tensor, temperature: Sequence[float], keys: Sequence[int],
                    steps: Sequence[int]) -> list:
        """The same from host lists, returning host integers."""
        device = logits.device
        if not any(value > 0 for value in temperature):
            return ops.argmax(logits).cpu().tolist()
        return self.select(logits,
                           torch.tensor(list(temperature), dtype=torch.float32, device=device),
                           torch.tensor(list(keys), dtype=torch.int64, device=device),
                           torch.tensor(list(steps), dtype=torch.int32, device=device)).cpu().tolist()
