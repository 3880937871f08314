"""The cache: a slot for each sequence of a batch, keys and values for each layer.

The reference keeps one heap state object per request with per-layer K and V of a
fixed capacity, a position, and rewind by moving the position
(src/kidi/model/gemma4.cpp:472-518,545-560); layers reach their cache through a
layer-to-cache map so that several layers can share one and layers with different
geometry have their own (src/kidi/model/gemma4.cpp:149-155,503-505).

Here the storage is paged. A slot is a small integer a sequence holds from its first
step until it ends. Each position of the run order (a "schedule entry") asks for
what its mixer needs:

* `KVRequest(kv_heads, head_dim, window)`: keys and values per token. Entries with
  equal requests form a group with storage of its own,
  K and V `[entries, pages, kv_heads, page_size, head_dim]`. A sequence holds pages of
  `page_size` tokens in each group, found through the group's block table
  `[slots, pages_per_sequence]`. With `window=None` a sequence holds a page for every
  `page_size` tokens it has; with a window it holds a ring of
  `ceil(window / page_size)` pages at most, and token `u` lives in ring row
  `u mod (ring_pages * page_size)`.
* `StateRequest(shape, dtype)`: per-sequence state of fixed size, stored
  `[entries, slots + 1, *shape]` and zeroed when a slot is handed out.

The last row of every state tensor and of every block table belongs to the padding slot
(`padding_slot`, one past the slots that are handed out): a captured decode step has a
fixed number of rows, and the sequences beyond the live ones carry that slot, so that a
mixer which updates "the state of every sequence of the step" writes, for them, where
nothing is ever read.

The budget is a number of tokens (`max_tokens`): the most that live sequences hold at
any time, each sequence's count rounded up to a whole page. Slots and pages are
given back by `release` and handed out again.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..errors import invalid_argument, runtime_error
from .allocator import IdAllocator

PAGE_SIZE = 64


@dataclasses.dataclass(frozen=True)
class KVRequest:
    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclasses.dataclass(frozen=True)
class StateRequest:
    shape: Tuple[int, ...]
    dtype: Optional[torch.dtype] = None  # None: the engine's activation dtype


CacheRequest = Union[KVRequest, StateRequest, None]


class KVGroup:
    """Storage and block table of the entries that share one `KVRequest`."""

    def __init__(self, request: KVRequest, entries: List[int], n_slots: int, n_pages: int, page_size: int,
                 max_positions: int, dtype: torch.dtype, device: torch.device):
        self.request = request
        self.entries = entries
        self.page_size = page_size
        full_pages = -(-max_positions // page_size)
        if request.window is None:
            self.ring_pages = 0  # 0: not a ring
            self.pages_per_sequence = min(full_pages, n_pages)
        else:
            if request.window <= 0:
                raise invalid_argument("an attention window must be positive")
            self.ring_pages = min(-(-request.window // page_size), full_pages)
            self.pages_per_sequence = self.ring_pages
            n_pages = min(n_pages, n_slots * self.ring_pages)
        self.n_pages = n_pages
        self.pool = IdAllocator(n_pages, "cache page")
        shape = (len(entries), n_pages, request.kv_heads, page_size, request.head_dim)
        # Rows of a page beyond a sequence's length are loaded with their tile and multiplied by
        # a zero probability, so the values there have to be finite (keys need not be: a masked
        # score is replaced whatever it was). The pools start zero-filled, and the values of a
        # page that has been used are cleared when it is handed out again (`clear_used`): what
        # an earlier sequence left, were it ever an infinity or a NaN, must not reach the next.
        self.keys = torch.zeros(shape, dtype=dtype, device=device)
        self.values = torch.zeros(shape, dtype=dtype, device=device)
        self.used = np.zeros(n_pages, dtype=bool)       # pages that have been handed out before
        # One row more than there are slots: the padding slot's (all zeros, never filled in).
        self.table_host = np.zeros((n_slots + 1, self.pages_per_sequence), dtype=np.int32)
        self.table = torch.zeros((n_slots + 1, self.pages_per_sequence), dtype=torch.int32, device=device)
        self.pages: Dict[int, List[int]] = {}
        self._dirty: set = set()

    @property
    def ring_tokens(self) -> int:
        return self.ring_pages * self.page_size

    def clear_used(self, pages: Sequence[int]) -> None:
        """Clears the values of those of `pages` that were handed out before, as runs of
        consecutive pages (on the current stream, before the step that writes them)."""
        again = sorted(page for page in pages if self.used[page])
        self.used[list(pages)] = True
        start = 0
        while start < len(again):
            stop = start + 1
            while stop < len(again) and again[stop] == again[stop - 1] + 1:
                stop += 1
            self.values[:, again[start]:again[stop - 1] + 1].zero_()
            start = stop

    def pages_for(self, length: int) -> int:
        needed = -(-length // self.page_size)
        return min(needed, self.ring_pages) if self.ring_pages else needed

    def bytes(self) -> int:
        return 2 * self.keys.numel() * self.keys.element_size()


class StateGroup:
    def __init__(self, request: StateRequest, entries: List[int], n_slots: int, dtype: torch.dtype,
                 device: torch.device):
        self.request = request
        self.entries = entries
        # One row more than there are slots: the padding slot's, which anything may be written to.
        self.storage = torch.zeros((len(entries), n_slots + 1, *request.shape), dtype=request.dtype or dtype,
                                   device=device)

    def bytes(self) -> int:
        return self.storage.numel() * self.storage.element_size()


@dataclasses.dataclass(frozen=True)
class StateSnapshot:
    """The fixed-size state of one slot at one length (see `SequenceCache.snapshot_state`)."""

    slot: int
    length: int
    tensors: list


@dataclasses.dataclass(frozen=True)
class KVView:
    """What one schedule entry's mixer sees of the cache."""

    group: KVGroup
    index: int  # the entry's index inside the group

    @property
    def keys(self) -> torch.Tensor:
        return self.group.keys[self.index]

    @property
    def values(self) -> torch.Tensor:
        return self.group.values[self.index]

    @property
    def table(self) -> torch.Tensor:
        return self.group.table

    @property
    def page_size(self) -> int:
        return self.group.page_size

    @property
    def ring_pages(self) -> int:
        return self.group.ring_pages


class SequenceCache:
    def __init__(self, requests: Sequence[Sequence[CacheRequest]], *, max_tokens: int, max_positions: int,
                 dtype: torch.dtype, device: torch.device, page_size: int = PAGE_SIZE,
                 max_slots: Optional[int] = None, cache_from: Optional[Sequence[Optional[int]]] = None):
        """`requests[e]` lists what schedule entry `e` asks for (a mixer may ask for
        several things, or nothing). `cache_from[e]`, if not None, names an earlier
        entry whose views entry `e` gets instead of storage of its own."""
        if page_size <= 0 or page_size & (page_size - 1):
            raise invalid_argument("the page size must be a power of two")
        if max_tokens <= 0:
            raise invalid_argument("the cache needs a positive token budget")
        self.page_size = page_size
        self.max_positions = max_positions
        self.max_tokens = -(-max_tokens // page_size) * page_size
        n_pages = self.max_tokens // page_size
        self.n_slots = min(n_pages, max_slots) if max_slots else n_pages
        self.slots = IdAllocator(self.n_slots, "cache slot")
        self.padding_slot = self.n_slots          # never handed out: what padding sequences of a captured step carry
        self.lengths: Dict[int, int] = {}
        self.dtype, self.device = dtype, device
        cache_from = list(cache_from) if cache_from is not None else [None] * len(requests)

        kv_groups: Dict[KVRequest, List[Tuple[int, int]]] = {}
        state_groups: Dict[StateRequest, List[Tuple[int, int]]] = {}
        for entry, wanted in enumerate(requests):
            if cache_from[entry] is not None:
                continue
            for position, request in enumerate(wanted):
                if isinstance(request, KVRequest):
                    kv_groups.setdefault(request, []).append((entry, position))
                elif isinstance(request, StateRequest):
                    state_groups.setdefault(request, []).append((entry, position))
                elif request is not None:
                    raise invalid_argument(f"entry {entry} asks the cache for {request!r}")
        self.kv_groups: List[KVGroup] = []
        self.state_groups: List[StateGroup] = []
        self._views: Dict[Tuple[int, int], object] = {}
        for request, users in kv_groups.items():
            group = KVGroup(request, [entry for entry, _ in users], self.n_slots, n_pages, page_size,
                            max_positions, dtype, device)
            self.kv_groups.append(group)
            for index, user in enumerate(users):
                self._views[user] = KVView(group, index)
        for request, users in state_groups.items():
            group = StateGroup(request, [entry for entry, _ in users], self.n_slots, dtype, device)
            self.state_groups.append(group)
            for index, user in enumerate(users):
                self._views[user] = group.storage[index]
        self._n_requests = [len(wanted) for wanted in requests]
        self._cache_from = cache_from

    # ------------------------------------------------------------------ views
    def views(self, entry: int) -> List[object]:
        """The views of schedule entry `entry`, in the order of its requests: a
        `KVView` per `KVRequest`, a tensor `[slots + 1, *shape]` per `StateRequest` (its last
        row is the padding slot's)."""
        source = self._cache_from[entry]
        if source is not None:
            if source >= entry or self._cache_from[source] is not None:
                raise invalid_argument(f"entry {entry} may read the cache of an earlier entry that owns one")
            return self.views(source)
        return [self._views.get((entry, position)) for position in range(self._n_requests[entry])]

    # ------------------------------------------------------------------ slots
    def acquire(self) -> int:
        slot = self.slots.acquire()
        self.lengths[slot] = 0
        for group in self.kv_groups:
            group.pages[slot] = []
        for group in self.state_groups:
            group.storage[:, slot].zero_()
        return slot

    def release(self, slot: int) -> None:
        self.slots.release(slot)  # raises on a slot that is not held
        del self.lengths[slot]
        for group in self.kv_groups:
            group.pool.release_many(group.pages.pop(slot))

    def length(self, slot: int) -> int:
        if slot not in self.lengths:
            raise invalid_argument(f"cache slot {slot} is not held")
        return self.lengths[slot]

    def can_hold(self, growth: Sequence[Tuple[int, int]]) -> bool:
        """Whether every (slot, new length) of `growth` fits the free pages."""
        for group in self.kv_groups:
            needed = sum(max(0, group.pages_for(length) - len(group.pages[slot])) for slot, length in growth)
            if needed > group.pool.free_count:
                return False
        return True

    def reserve(self, growth: Sequence[Tuple[int, int]]) -> None:
        """Makes room for each slot to hold `new length` tokens; all or nothing."""
        for slot, length in growth:
            if slot not in self.lengths:
                raise invalid_argument(f"cache slot {slot} is not held")
            if length < self.lengths[slot]:
                raise invalid_argument(f"slot {slot} holds {self.lengths[slot]} tokens and cannot shrink to {length}")
            if length > self.max_positions:
                raise invalid_argument(
                    f"a sequence of {length} tokens exceeds the positional capacity of {self.max_positions}")
        if not self.can_hold(growth):
            raise runtime_error(
                f"the cache is full: a budget of {self.max_tokens} tokens cannot hold this step "
                f"(each sequence's length is rounded up to {self.page_size})")
        for group in self.kv_groups:
            for slot, length in growth:
                held = group.pages[slot]
                extra = group.pages_for(length) - len(held)
                if extra > 0:
                    first = len(held)
                    held.extend(group.pool.acquire_many(extra))
                    group.clear_used(held[first:])
                    group.table_host[slot, first:len(held)] = held[first:]
                    group._dirty.add(slot)

    def commit(self, growth: Sequence[Tuple[int, int]]) -> None:
        for slot, length in growth:
            self.lengths[slot] = length

    def snapshot_state(self, slot: int) -> "StateSnapshot":
        """A copy of the slot's fixed-size state (every state group) as it is now, with the
        sequence's length: what `rewind` needs to come back to this point (keys and values
        need none: their rows beyond the length are simply forgotten)."""
        return StateSnapshot(slot, self.length(slot), [group.storage[:, slot].clone() for group in self.state_groups])

    def rewind(self, slot: int, length: int, state: Optional["StateSnapshot"] = None) -> None:
        """Forgets tokens beyond `length` (the reference's rewind moves the position,
        src/kidi/model/gemma4.cpp:545-560). Full-history groups give pages back; a ring
        cannot be rewound past what it overwrote. Fixed-size state cannot be computed
        backwards: a model that has some is rewound to a point of which `state` is the
        snapshot (`snapshot_state`, taken at that length)."""
        current = self.length(slot)
        if length < 0 or length > current:
            raise invalid_argument(f"cannot rewind slot {slot} from {current} to {length}")
        if state is not None and (state.slot != slot or state.length != length or
                                  len(state.tensors) != len(self.state_groups)):
            raise invalid_argument("the state snapshot is not of this slot at this length")
        for group in self.kv_groups:
            if group.ring_pages and current > group.ring_tokens and length < current:
                raise invalid_argument("a windowed cache that has wrapped cannot be rewound")
            keep = group.pages_for(length)
            held = group.pages[slot]
            group.pool.release_many(held[keep:])
            del held[keep:]
        if self.state_groups and length < current:
            if state is None:
                raise invalid_argument("fixed-size per-sequence state cannot be rewound without a snapshot "
                                       "taken at the length to return to")
            for group, saved in zip(self.state_groups, state.tensors):
                group.storage[:, slot].copy_(saved)
        self.lengths[slot] = length

    def flush_tables(self) -> None:
        """Copies block-table rows that changed since the last call to the device."""
        for group in self.kv_groups:
            for slot in sorted(group._dirty):
                row = torch.from_numpy(group.table_host[slot])
                group.table[slot].copy_(row, non_blocking=False)
            group._dirty.clear()

    # ------------------------------------------------------------- accounting
    def bytes(self) -> int:
        return sum(group.bytes() for group in self.kv_groups) + sum(group.bytes() for group in self.state_groups)

    def held_tokens(self) -> int:
        return sum(-(-length // self.page_size) * self.page_size for length in self.lengths.values())

    def check(self) -> None:
        """Raises if a slot or a page is lost, held twice or inconsistent."""
        self.slots.check()
        if set(self.lengths) != self.slots.held:
            raise runtime_error("slot lengths and held slots disagree")
        for group in self.kv_groups:
            group.pool.check()
            seen: List[int] = []
            for slot, pages in group.pages.items():
                if slot not in self.lengths:
                    raise runtime_error(f"pages are kept for slot {slot}, which is not held")
                if len(pages) < group.pages_for(self.lengths[slot]):
                    raise runtime_error(f"slot {slot} holds fewer pages than its length needs")
                seen.extend(pages)
            if len(seen) != len(set(seen)):
                raise runtime_error("a cache page belongs to two sequences")
            if set(seen) != group.pool.held:
                raise runtime_error("held pages and the pages of sequences disagree")
