"""What one step runs: the packed rows of a batch and where each row lies.

A step takes B sequences that each bring T_b >= 1 new tokens (their whole prompts, or
one decoded token each) and runs the sum of T_b rows as one packed batch, the way the
reference packs several segments into one row set with positions restarting per
segment (src/kidi/model/qwen3.cpp:206-238, src/kidi/layers/qwen3.cpp:58-98). This
module builds, on the host and without a GPU, the integer tables every kernel reads:

* per row: the sequence it belongs to (`row_seq`) and its absolute position
  (`row_pos`);
* per sequence: its cache slot, the tokens it held before the step (`seq_start`), the
  tokens it brings (`seq_len`) and its first packed row (`seq_row0`);
* the packed rows whose logits are wanted (`want_rows`).

Validation happens here, before anything is launched (as
src/kidi/model/gemma4.cpp:989-995 does): token ids in range, distinct slots, wanted
places inside the new tokens.
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional, Sequence

import numpy as np

from ..errors import invalid_argument


@dataclasses.dataclass
class StepBatch:
    """The caller's view of a step. `want[b]` lists places among `tokens[b]` whose
    logits are returned; None means the last token of every sequence."""

    slots: Sequence[int]
    tokens: Sequence[Sequence[int]]
    want: Optional[Sequence[Sequence[int]]] = None


@dataclasses.dataclass
class StepPlan:
    n_rows: int
    n_seqs: int
    n_want: int
    max_new: int          # longest T_b
    max_total: int        # longest seq_start + T_b
    is_decode: bool       # every sequence brings exactly one token
    tokens: np.ndarray    # int32 [n_rows]
    row_seq: np.ndarray   # int32 [n_rows]
    row_pos: np.ndarray   # int32 [n_rows]
    seq_slot: np.ndarray  # int32 [n_seqs]
    seq_start: np.ndarray  # int32 [n_seqs]
    seq_len: np.ndarray   # int32 [n_seqs]
    seq_row0: np.ndarray  # int32 [n_seqs]
    want_rows: np.ndarray  # int32 [n_want]

    FIELDS = ("tokens", "row_seq", "row_pos", "seq_slot", "seq_start", "seq_len", "seq_row0", "want_rows")

    def packed(self) -> np.ndarray:
        """All tables in one int32 array (one host-to-device copy), each field padded
        to a multiple of 4 entries so that it starts on a 16-byte boundary."""
        parts = []
        for name in self.FIELDS:
            field = getattr(self, name)
            parts.append(field)
            if field.size % 4:
                parts.append(np.zeros(4 - field.size % 4, dtype=np.int32))
        return np.concatenate(parts) if parts else np.zeros(0, dtype=np.int32)

    def offsets(self) -> dict:
        offsets, cursor = {}, 0
        for name in self.FIELDS:
            size = getattr(self, name).size
            offsets[name] = (cursor, size)
            cursor += size + (-size % 4)
        return offsets


def build_plan(batch: StepBatch, starts: Sequence[int], vocab_size: int) -> StepPlan:
    """`starts[b]` is the number of tokens sequence b holds in the cache already."""
    n_seqs = len(batch.slots)
    if n_seqs == 0:
        raise invalid_argument("a step needs at least one sequence")
    if len(batch.tokens) != n_seqs or len(starts) != n_seqs:
        raise invalid_argument("a step needs tokens for every sequence")
    if len(set(batch.slots)) != n_seqs:
        raise invalid_argument("a step names a cache slot twice")
    if batch.want is not None and len(batch.want) != n_seqs:
        raise invalid_argument("'want' must have an entry for every sequence")
    lengths = [len(tokens) for tokens in batch.tokens]
    if min(lengths) < 1:
        raise invalid_argument("every sequence of a step brings at least one token")
    n_rows = sum(lengths)
    tokens = np.empty(n_rows, dtype=np.int64)
    row_seq = np.empty(n_rows, dtype=np.int32)
    row_pos = np.empty(n_rows, dtype=np.int32)
    seq_row0 = np.zeros(n_seqs, dtype=np.int32)
    want_rows: List[int] = []
    cursor = 0
    for index, (new, start) in enumerate(zip(batch.tokens, starts)):
        count = len(new)
        seq_row0[index] = cursor
        tokens[cursor:cursor + count] = np.asarray(new, dtype=np.int64)
        row_seq[cursor:cursor + count] = index
        row_pos[cursor:cursor + count] = np.arange(start, start + count, dtype=np.int32)
        if batch.want is None:
            want_rows.append(cursor + count - 1)
        else:
            for place in batch.want[index]:
                if not isinstance(place, (int, np.integer)) or place < 0 or place >= count:
                    raise invalid_argument(f"wanted place {place!r} lies outside the {count} new tokens")
                want_rows.append(cursor + int(place))
        cursor += count
    if tokens.min() < 0 or tokens.max() >= vocab_size:
        bad = int(tokens[(tokens < 0) | (tokens >= vocab_size)][0])
        raise invalid_argument(f"token id {bad} lies outside the vocabulary of {vocab_size}")
    seq_start = np.asarray(starts, dtype=np.int32)
    seq_len = np.asarray(lengths, dtype=np.int32)
    return StepPlan(
        n_rows=n_rows, n_seqs=n_seqs, n_want=len(want_rows),
        max_new=int(seq_len.max()), max_total=int((seq_start + seq_len).max()),
        is_decode=bool((seq_len == 1).all()),
        tokens=tokens.astype(np.int32), row_seq=row_seq, row_pos=row_pos,
        seq_slot=np.asarray(batch.slots, dtype=np.int32), seq_start=seq_start, seq_len=seq_len,
        seq_row0=seq_row0, want_rows=np.asarray(want_rows, dtype=np.int32),
    )
