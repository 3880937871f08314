"""The decode step of a batch, captured once as a CUDA graph and replayed.

A decode step launches a few hundred small kernels; launching them one by one from
the host costs as much as running them. The reference captures its recorded decode
step into a `cudaGraph` and replays it, with pointer-stable tables for what changes
between steps (src/kidi/runtime/cuda/operators.cpp:202-277,292,438-471). Here a
`DecodeSession` owns static device buffers for a batch of up to `capacity` rows: the
step's integer tables, the sampling parameters and the selected tokens. The captured
graph runs the model's ordinary forward pass over those buffers, selects a token per
row on the device, and advances tokens and positions for the next step. Between
replays the host only rewrites the buffers (one copy) when the set of live sequences
changes, and reads the selected tokens back. The tokens a step selects are its
successor's inputs where they lie on the device, so the host may submit the next step
before it has read the last one's tokens (the reference's decode-ahead with device tokens
and an asynchronous read-back into pinned memory, src/kidi/inference/generator.cpp:1044-1093).

Rows beyond the live sequences are padding: their `row_seq` is -1, so they write
nothing to the cache and attend to nothing; what the other kernels compute for them is
never read. The rule for every part that keeps something per sequence: a row whose
`row_seq` is negative touches neither keys, values nor state of any slot. As a net
under that rule the padding sequences carry the cache's padding slot in `seq_slot`
(the last row of every state tensor and block table), never a slot that a live
sequence may hold. The host tables of the step's `plan` are placeholders here (the
graph is captured once): a part that is to run in a captured step reads `ctx.tables`.
"""
from __future__ import annotations

import gc
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..errors import invalid_argument
from ..kernels import ops
from .plan import StepPlan


class DecodeSession:
    FIELDS = ("tokens", "row_seq", "row_pos", "seq_slot", "seq_start", "seq_len", "seq_row0", "want_rows", "steps")
    READBACK_DEPTH = 4

    def __init__(self, engine, capacity: int, sampler, *, longest: Optional[int] = None):
        from .engine import DeviceTables, StepContext
        self.engine = engine
        self.capacity = capacity
        self.sampler = sampler
        device = engine.device
        padded = -(-capacity // 4) * 4
        self._padded = padded
        # One int32 buffer: the FIELDS, then temperature (float32 bits), then keys (int64 as two words).
        words = padded * (len(self.FIELDS) + 1 + 2)
        self.buffer = torch.zeros(words, dtype=torch.int32, device=device)
        self.staging = torch.zeros(words, dtype=torch.int32).pin_memory()
        self._host = self.staging.numpy()
        offsets = {name: (index * padded, capacity) for index, name in enumerate(self.FIELDS)}
        self.tables = DeviceTables(self.buffer, offsets)
        base = len(self.FIELDS) * padded
        self.temperature = self.buffer[base:base + capacity].view(torch.float32)
        self.keys = self.buffer[base + padded:base + padded + 2 * capacity].view(torch.int64)
        self._offsets = offsets
        self._temperature_at = base
        self._keys_at = base + padded
        self.selected = torch.zeros(capacity, dtype=torch.int32, device=device)
        # Read-back buffers in pinned memory, used in turn: a step's tokens stay readable while
        # the steps submitted after it run.
        self._readback = [torch.zeros(capacity, dtype=torch.int32).pin_memory() for _ in range(self.READBACK_DEPTH)]
        self._readback_views = [buffer.numpy() for buffer in self._readback]
        self._readback_done = [torch.cuda.Event() for _ in range(self.READBACK_DEPTH)]
        self._submitted = 0            # steps submitted since the session was made
        self.tokens_host = torch.zeros(capacity, dtype=torch.int32).pin_memory()
        self._tokens_host_view = self.tokens_host.numpy()
        self.logits: Optional[torch.Tensor] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.live = 0
        rows = np.arange(capacity, dtype=np.int32)
        self._plan = StepPlan(
            n_rows=capacity, n_seqs=capacity, n_want=capacity, max_new=1,
            max_total=longest or engine.spec.max_positions, is_decode=True,
            tokens=rows * 0, row_seq=rows, row_pos=rows * 0, seq_slot=rows * 0 + engine.cache.padding_slot,
            seq_start=rows * 0,
            seq_len=rows * 0 + 1, seq_row0=rows, want_rows=rows)
        # Launch dimensions that depend on the sequence length (the key splits of decode
        # attention, chosen by each attention part for its own geometry) are fixed when the graph
        # is captured, from `max_total`: the longest sequence this session may come to hold.
        self._context = StepContext(self._plan, self.tables, engine.cache, engine.dtype, device, engine._workspaces)
        self._stream = torch.cuda.Stream(device=device)

    # ------------------------------------------------------------------ set-up
    def load(self, slots: Sequence[int], tokens: Sequence[int], temperature: Sequence[float], keys: Sequence[int],
             steps: Sequence[int]) -> None:
        """Sets the live sequences: row r continues the sequence in `slots[r]` with the
        input token `tokens[r]` at the position the cache says it has reached."""
        live = len(slots)
        if live < 1 or live > self.capacity:
            raise invalid_argument(f"a decode session of {self.capacity} rows cannot hold {live} sequences")
        if len(set(slots)) != live:
            raise invalid_argument("a step names a cache slot twice")
        cache = self.engine.cache
        starts = [cache.length(slot) for slot in slots]
        host, padded, capacity = self._host, self._padded, self.capacity

        def field(name):
            begin = self._offsets[name][0]
            return host[begin:begin + capacity]

        field("tokens")[:] = 0
        field("tokens")[:live] = tokens
        field("row_seq")[:] = -1
        field("row_seq")[:live] = np.arange(live, dtype=np.int32)
        field("row_pos")[:] = 0
        field("row_pos")[:live] = starts
        field("seq_slot")[:] = cache.padding_slot
        field("seq_slot")[:live] = slots
        field("seq_start")[:] = 0
        field("seq_start")[:live] = starts
        field("seq_len")[:] = 1
        field("seq_row0")[:] = np.arange(capacity, dtype=np.int32)
        field("want_rows")[:] = np.arange(capacity, dtype=np.int32)
        field("steps")[:] = 0
        field("steps")[:live] = steps
        host[self._temperature_at:self._temperature_at + capacity].view(np.float32)[:] = 0.0
        host[self._temperature_at:self._temperature_at + live].view(np.float32)[:] = temperature
        host[self._keys_at:self._keys_at + 2 * capacity].view(np.int64)[:] = 0
        host[self._keys_at:self._keys_at + 2 * live].view(np.int64)[:] = keys
        self.buffer.copy_(self.staging, non_blocking=True)
        self.uploaded_bytes = self.staging.numel() * self.staging.element_size()
        torch.cuda.current_stream().synchronize()  # the staging buffer may be rewritten after this
        self.live = live
        self.slots = list(slots)
        self.positions = list(starts)

    # -------------------------------------------------------------------- step
    def _forward(self) -> None:
        engine = self.engine
        self.logits = engine.model.forward(self._context)
        self.sampler.select(self.logits, self.temperature, self.keys, self.tables.steps, out=self.selected)
        ops.advance_decode(self.tables.tokens, self.selected, self.tables.row_seq, self.tables.row_pos,
                           self.tables.seq_start, self.tables.steps, engine.vocab_size)

    def _capture(self) -> None:
        """Runs the step once with every row padded (nothing is written to the cache), so
        that kernels are compiled and configured, then captures it."""
        saved = self.buffer.clone()
        begin = self._offsets["row_seq"][0]
        self.buffer[begin:begin + self.capacity] = -1
        begin = self._offsets["seq_slot"][0]
        self.buffer[begin:begin + self.capacity] = self.engine.cache.padding_slot
        torch.cuda.synchronize(self.engine.device)
        with torch.cuda.stream(self._stream):
            self._forward()
        self._stream.synchronize()
        self.buffer.copy_(saved)
        torch.cuda.synchronize(self.engine.device)
        self.graph = torch.cuda.CUDAGraph()
        before = ops.launch_count
        # Nothing but the step's own launches may touch CUDA while it is captured. The
        # collector is held off (a finaliser of an unrelated object that frees device or
        # pinned memory in the middle of the capture would invalidate it), and the capture
        # is thread-local, as the reference's is (src/kidi/runtime/cuda/operators.cpp:262-276).
        was_enabled = gc.isenabled()
        gc.collect()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph, stream=self._stream, capture_error_mode="thread_local"):
                self._forward()
        finally:
            if was_enabled:
                gc.enable()
        self.kernels_per_step = ops.launch_count - before   # this package's kernels in one replay
        self.buffer.copy_(saved)
        torch.cuda.synchronize(self.engine.device)
        # The graph holds the addresses of the scratch buffers it was captured with; they
        # must outlive it even if the engine later replaces them with larger ones.
        self._captured_workspaces = dict(self.engine._workspaces)

    def reserve(self, steps: int = 1) -> None:
        """Makes sure the cache has room for `steps` more tokens of every live sequence."""
        cache = self.engine.cache
        cache.reserve([(slot, position + steps) for slot, position in zip(self.slots, self.positions)])
        cache.flush_tables()

    def launch(self) -> None:
        """One decode step on the device (no host synchronisation). The caller has reserved room."""
        if self.graph is None:
            self._capture()
        self.graph.replay()
        self.positions = [position + 1 for position in self.positions]
        self.engine.cache.commit(list(zip(self.slots, self.positions)))

    def submit(self, tokens: Optional[Sequence[int]] = None) -> int:
        """Submits one decode step without waiting for it and returns a ticket for `read`.
        Without `tokens` the step's inputs are the tokens the previous step selected, where
        they lie on the device; with `tokens` (host integers, one per live sequence) they are
        copied from pinned host memory first. At most READBACK_DEPTH - 1 steps may be
        submitted beyond the last one read."""
        self.reserve(1)
        if tokens is not None:
            self._tokens_host_view[:self.live] = tokens
            self.tables.tokens[:self.live].copy_(self.tokens_host[:self.live], non_blocking=True)
        self.launch()
        ticket = self._submitted
        self._submitted += 1
        turn = ticket % self.READBACK_DEPTH
        self._readback[turn].copy_(self.selected, non_blocking=True)
        self._readback_done[turn].record()
        return ticket

    def read(self, ticket: int) -> List[int]:
        """Waits for the step of `ticket` and returns the token it selected for every live
        sequence."""
        if not self._submitted - self.READBACK_DEPTH < ticket < self._submitted:
            raise invalid_argument("this step's tokens are no longer kept (too many steps were submitted since)")
        turn = ticket % self.READBACK_DEPTH
        self._readback_done[turn].synchronize()
        return self._readback_views[turn][:self.live].tolist()

    def step(self, tokens: Optional[Sequence[int]] = None) -> List[int]:
        """One decode step, waited for: the selected token of every live sequence."""
        return self.read(self.submit(tokens))
