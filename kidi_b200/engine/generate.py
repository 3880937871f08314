"""The generation loop above the step function.

Requests are cut into batches that start together (`search.plan_batches`). A batch's
prompts, of unequal lengths, run in one step (or in chunks of `prefill_chunk_size`
tokens per sequence); the first token of every sequence is selected from the logits at
its prompt's last token; then the live sequences go on by one token per step. A
sequence that meets a stop token or its limit leaves the batch at once and gives its
slot and pages back; the batch ends when none is left, and the next batch starts on
the same slots. Results come back in the order of the requests.

This is the reference's `Generator::generate_batch` over `Decoder::generate_batch`
(src/kidi/inference/generator.cpp:539-641, src/kidi/inference/decoder.cpp:346-401:
per step the live rows, one token each, `accept` per row, finished rows leave), with
its limits (src/kidi/inference/generator.cpp:136-140,438-445: `maximum_new_tokens` 0 means
the default of 8192, `context_size` 0 means min(max_position_embeddings, 16384), a prompt
and its new tokens must fit the context). Unlike the reference, which prefills each
prompt alone (src/kidi/inference/generator.cpp:573-604), the prompts of a batch share one step.

Decoding runs one step ahead of the host (the reference's decode-ahead,
src/kidi/inference/generator.cpp:1044-1093): a step's selected tokens are its successor's
inputs where they lie on the device, so the loop submits step n+1 before it reads the
tokens of step n, and the read-back and the stop test overlap the device's work. A step
is only submitted ahead when no sequence can reach its length limit in the step before
it; when a stop token ends a sequence after all, the step that already ran is still
right for the others (a sequence's tokens do not depend on its neighbours), so its
tokens are kept for them and only the ended sequence's extra token is dropped.
"""
from __future__ import annotations

import dataclasses
import time
from typing import Callable, Dict, List, Optional, Sequence

from ..errors import invalid_argument
from .plan import StepBatch
from .search import Generation, SequenceState, plan_batches

DEFAULT_MAX_NEW_TOKENS = 8192
DEFAULT_CONTEXT_LIMIT = 16384
DEFAULT_MAX_ACTIVE = 4   # the command line's default, as the reference's (src/kidi/cli/main.cpp:905-958);
                         # `Engine.generate` without `max_active` takes as many as the cache has slots for
MAX_KEPT_SESSIONS = 6    # captured decode steps an engine keeps (the least recently used goes first)


@dataclasses.dataclass
class GenerationOptions:
    max_new_tokens: int = 0          # 0: the default (8192, or what the context leaves)
    context_size: int = 0            # 0: min(max_position_embeddings, 16384)
    prefill_chunk_size: int = 0      # 0: a prompt runs whole in one step
    temperature: float = 0.0         # 0: greedy
    seed: int = 0
    ignore_eos: bool = False
    stop_ids: Sequence[int] = ()     # in addition to the model's end tokens
    max_active: int = DEFAULT_MAX_ACTIVE
    use_graph: bool = True           # replay decode steps as a CUDA graph


@dataclasses.dataclass
class GenerationStats:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    decode_steps: int = 0
    batches: int = 0
    prefill_ns: int = 0
    decode_ns: int = 0
    time_to_first_token_ns: int = 0
    generation_ns: int = 0
    host_to_device_bytes: int = 0   # copied up while decoding (the tables of a batch, when a session is loaded)


class Backend:
    """What the loop needs from an engine; tests substitute a fake one.

    acquire() -> slot; release(slot); prefill(slots, chunks, select, ...) -> the first
    tokens of the sequences whose prompt the chunk ends; open_decode(slots, tokens, ...) ->
    a session with submit() -> ticket (one more step for every sequence, not waited for,
    fed with the tokens of the step before it) and read(ticket) -> that step's tokens."""


class EngineBackend(Backend):
    def __init__(self, engine, sampler, use_graph: bool = True):
        self.engine, self.sampler, self.use_graph = engine, sampler, use_graph
        self._sessions: Dict[int, object] = {}
        self.vocab_size = engine.vocab_size
        self.max_positions = engine.spec.max_positions
        self.token_budget = engine.cache.max_tokens
        self.page = engine.cache.page_size
        self.max_slots = engine.cache.n_slots

    def acquire(self) -> int:
        return self.engine.acquire()

    def release(self, slot: int) -> None:
        self.engine.release(slot)

    def prefill(self, slots, chunks, select, temperature, keys, steps):
        """Runs `chunks[b]` for the sequence in `slots[b]`; `select[b]` says whether the
        chunk ends the prompt. Returns the first token of the sequences it does."""
        want = [[len(chunk) - 1] if chosen else [] for chunk, chosen in zip(chunks, select)]
        logits = self.engine.step(StepBatch(list(slots), [list(chunk) for chunk in chunks], want))
        if not any(select):
            return []
        pick = [index for index, chosen in enumerate(select) if chosen]
        return self.sampler.select_host(logits, [temperature[i] for i in pick], [keys[i] for i in pick],
                                        [steps[i] for i in pick])

    def open_decode(self, slots, tokens, temperature, keys, steps, longest):
        from .decode_graph import DecodeSession
        if not self.use_graph:
            return _EagerDecode(self, slots, tokens, temperature, keys, steps)
        capacity = 1
        while capacity < len(slots):
            capacity *= 2
        longest = min(longest, self.max_positions)
        # A captured step freezes launch choices that depend on the longest sequence (the key
        # splits of decode attention): a call with other choices gets a capture of its own.
        key = (capacity, self.engine.model.launch_signature(capacity, longest))
        session = self._sessions.pop(key, None)
        if session is None:
            session = DecodeSession(self.engine, capacity, self.sampler, longest=longest)
            while len(self._sessions) >= MAX_KEPT_SESSIONS:
                self._sessions.pop(next(iter(self._sessions)))
        self._sessions[key] = session          # most recently used last
        session.load(slots, tokens, temperature, keys, steps)
        return session


class _EagerDecode:
    """Decode steps through `Engine.step`, one launch at a time (no graph). A submitted step
    runs when its tokens are asked for: every step needs its predecessor's tokens on the host."""

    def __init__(self, backend, slots, tokens, temperature, keys, steps):
        self.backend, self.slots, self.tokens = backend, list(slots), list(tokens)
        self.temperature, self.keys, self.steps = list(temperature), list(keys), list(steps)
        self._submitted, self._results = 0, {}

    def submit(self) -> int:
        self._submitted += 1
        return self._submitted - 1

    def read(self, ticket: int) -> List[int]:
        engine, sampler = self.backend.engine, self.backend.sampler
        while len(self._results) <= ticket:
            logits = engine.step(StepBatch(self.slots, [[token] for token in self.tokens], None))
            self.tokens = sampler.select_host(logits, self.temperature, self.keys, self.steps)
            self.steps = [step + 1 for step in self.steps]
            self._results[len(self._results)] = list(self.tokens)
        return self._results[ticket]


def generate(backend: Backend, prompts: Sequence[Sequence[int]], options: GenerationOptions,
             stop_ids: Sequence[int] = (), max_tokens: Optional[Sequence[Optional[int]]] = None,
             stats: Optional[GenerationStats] = None,
             on_finished: Optional[Callable[[int, Generation], None]] = None) -> List[Generation]:
    """Generates for every prompt (lists of token ids) and returns `Generation`s in the
    order of the prompts. `max_tokens[i]`, if given, limits request i's new tokens."""
    stats = stats if stats is not None else GenerationStats()
    started = time.perf_counter_ns()
    count = len(prompts)
    context = options.context_size or min(backend.max_positions, DEFAULT_CONTEXT_LIMIT)
    if context > backend.max_positions:
        raise invalid_argument(f"context size {context} exceeds the model's {backend.max_positions} positions")
    if options.temperature < 0 or options.prefill_chunk_size < 0 or options.max_active < 1:
        raise invalid_argument("temperature and chunk size must not be negative; max_active must be positive")
    limits: List[int] = []
    for index, prompt in enumerate(prompts):
        length = len(prompt)
        if length < 1 or length >= context:
            raise invalid_argument(f"request {index}: a prompt of {length} tokens must be non-empty and shorter "
                                   f"than the context of {context}")
        asked = max_tokens[index] if max_tokens is not None and max_tokens[index] else options.max_new_tokens
        if asked:
            if asked < 0 or asked > context - length:
                raise invalid_argument(f"request {index}: prompt and generation must fit the context "
                                       f"({length} + {asked} > {context})")
            limits.append(int(asked))
        else:
            limits.append(min(DEFAULT_MAX_NEW_TOKENS, context - length))
        if min(prompt) < 0 or max(prompt) >= backend.vocab_size:
            raise invalid_argument(f"request {index}: a token id lies outside the vocabulary of {backend.vocab_size}")
    stops = tuple(dict.fromkeys([*stop_ids, *options.stop_ids]))
    batches = plan_batches([len(p) for p in prompts], limits, token_budget=backend.token_budget, page=backend.page,
                           max_active=min(options.max_active, backend.max_slots), max_positions=backend.max_positions)
    results: List[Optional[Generation]] = [None] * count
    first_token_seen = False
    for begin, end in batches:
        stats.batches += 1
        members = list(range(begin, end))
        states = {i: SequenceState(backend.vocab_size, limits[i], stops, options.ignore_eos) for i in members}
        slots = {i: backend.acquire() for i in members}

        def finish(index: int) -> None:
            backend.release(slots.pop(index))
            results[index] = states[index].result()
            stats.generated_tokens += len(results[index].token_ids)
            if on_finished is not None:
                on_finished(index, results[index])

        try:
            # ---- prompts: whole, or chunk by chunk; the step that ends a prompt selects its first token
            tick = time.perf_counter_ns()
            done = {i: 0 for i in members}
            chunk = options.prefill_chunk_size
            while any(done[i] < len(prompts[i]) for i in members):
                rows = [i for i in members if done[i] < len(prompts[i])]
                pieces = [list(prompts[i][done[i]:done[i] + chunk] if chunk else prompts[i][done[i]:]) for i in rows]
                closing = [done[i] + len(piece) >= len(prompts[i]) for i, piece in zip(rows, pieces)]
                chosen = backend.prefill([slots[i] for i in rows], pieces, closing,
                                         [options.temperature] * len(rows), rows, [0] * len(rows))
                for i, piece in zip(rows, pieces):
                    done[i] += len(piece)
                    stats.prompt_tokens += len(piece)
                for i, token in zip([i for i, closed in zip(rows, closing) if closed], chosen):
                    states[i].accept(token)
            now = time.perf_counter_ns()
            stats.prefill_ns += now - tick
            if not first_token_seen:
                stats.time_to_first_token_ns = now - started
                first_token_seen = True
            for i in [i for i in members if states[i].finished]:
                finish(i)
            # ---- one token per live sequence per step, submitted one step ahead of the host;
            # the session is reopened when a sequence leaves
            tick = time.perf_counter_ns()
            live = [i for i in members if not states[i].finished]
            session, ticket = None, None
            while live:
                if session is None:
                    longest = max(len(prompts[i]) + limits[i] for i in live)
                    session = backend.open_decode([slots[i] for i in live], [states[i].token for i in live],
                                                  [options.temperature] * len(live), live,
                                                  [states[i].steps for i in live], longest)
                    stats.host_to_device_bytes += getattr(session, "uploaded_bytes", 0)
                    ticket = session.submit()
                # The step ahead: only if the step in flight cannot end a sequence by its limit.
                ahead = session.submit() if all(states[i].steps + 1 < limits[i] for i in live) else None
                chosen = session.read(ticket)
                stats.decode_steps += 1
                for i, token in zip(live, chosen):
                    states[i].accept(token)
                if ahead is not None and any(states[i].finished for i in live):
                    # A stop token ended a sequence, and the step ahead has run for every row
                    # already: the other sequences keep its tokens, the ended one's is dropped.
                    chosen = session.read(ahead)
                    stats.decode_steps += 1
                    for i, token in zip(live, chosen):
                        if not states[i].finished:
                            states[i].accept(token)
                    ahead = None
                if any(states[i].finished for i in live):
                    for i in [i for i in live if states[i].finished]:
                        finish(i)
                    live = [i for i in live if not states[i].finished]
                    session, ticket = None, None
                else:
                    ticket = ahead if ahead is not None else session.submit()
            stats.decode_ns += time.perf_counter_ns() - tick
        finally:
            for index in list(slots):
                backend.release(slots.pop(index))
    stats.generation_ns += time.perf_counter_ns() - started
    return results  # type: ignore[return-value]
