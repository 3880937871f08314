"""The decisions of the generation loop, without a device.

`SequenceState` is the reference's `GreedyState` (src/kidi/inference/decoder.cpp:65-101)
for one sequence: every selected token counts as a step; an end or stop token ends the
sequence and is not appended; otherwise the token is appended; the sequence also ends
at `max_new_tokens`, and is then `truncated` when stopping on end tokens was on.
`ignore_eos` (the command line's --ignore-eos; `stop_on_eos=false` in
src/kidi/inference/decoder.cpp:12-15) switches every stop off. A selected token of -1
(no valid score: NaN, +inf or nothing finite) is an error, as in
src/kidi/inference/decoder.cpp:72-80.

`plan_batches` cuts a list of requests into batches that start together: as many
requests, in order, as fit the limit on live sequences and the cache's token budget,
each request counted with the most tokens it may come to hold, rounded up to a page.
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional, Sequence, Tuple

from ..errors import invalid_argument, runtime_error


@dataclasses.dataclass
class Generation:
    token_ids: List[int]
    decoder_steps: int
    finish_reason: str        # "stop" or "length"
    truncated: bool


class SequenceState:
    def __init__(self, vocab_size: int, max_new_tokens: int, stop_ids: Sequence[int], ignore_eos: bool):
        if max_new_tokens < 1:
            raise invalid_argument("a sequence needs room for at least one new token")
        if any(token < 0 or token >= vocab_size for token in stop_ids):
            raise invalid_argument("a stop token lies outside the vocabulary")
        self.vocab_size = vocab_size
        self.max_new_tokens = max_new_tokens
        self.stop_ids = frozenset(stop_ids)
        self.ignore_eos = ignore_eos
        self.token_ids: List[int] = []
        self.steps = 0
        self.finished = False
        self.ended = False     # finished by a stop token
        self.token: Optional[int] = None  # the last selected token (the next step's input)

    def is_stop(self, token: int) -> bool:
        return not self.ignore_eos and token in self.stop_ids

    def accept(self, token: int) -> None:
        if self.finished:
            raise invalid_argument("generation is already finished")
        if token < 0 or token >= self.vocab_size:
            raise runtime_error("the decoder returned invalid scores (no valid token could be selected)")
        self.token = token
        self.steps += 1
        self.ended = self.is_stop(token)
        if not self.ended:
            self.token_ids.append(token)
        self.finished = self.ended or self.steps == self.max_new_tokens

    def result(self) -> Generation:
        return Generation(list(self.token_ids), self.steps, "stop" if self.ended else "length",
                          truncated=not self.ended and not self.ignore_eos)


def round_up(value: int, unit: int) -> int:
    return -(-value // unit) * unit


def plan_batches(prompt_lengths: Sequence[int], max_new_tokens: Sequence[int], *, token_budget: int, page: int,
                 max_active: int, max_positions: int) -> List[Tuple[int, int]]:
    """[(first request, one past the last)] of consecutive batches. Raises when a
    request alone exceeds the budget or the positional capacity."""
    if max_active < 1:
        raise invalid_argument("at least one sequence must be active at a time")
    batches: List[Tuple[int, int]] = []
    begin, held, index = 0, 0, 0
    count = len(prompt_lengths)
    while index < count:
        if prompt_lengths[index] < 1:
            raise invalid_argument(f"request {index} has an empty prompt")
        most = prompt_lengths[index] + max_new_tokens[index] - 1  # the last new token is never fed back
        if most > max_positions or prompt_lengths[index] >= max_positions:
            raise invalid_argument(f"request {index}: {prompt_lengths[index]} prompt tokens plus "
                                   f"{max_new_tokens[index]} new ones exceed the positional capacity {max_positions}")
        need = round_up(most, page)
        if need > token_budget:
            raise invalid_argument(f"request {index} may come to hold {need} tokens; the cache holds {token_budget}")
        if index > begin and (held + need > token_budget or index - begin >= max_active):
            batches.append((begin, index))
            begin, held = index, 0
        held += need
        index += 1
    if count:
        batches.append((begin, count))
    return batches
