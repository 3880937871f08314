"""The generation loop's decisions, driven by a fake model (no GPU): batches of unequal
prompts, stop tokens, sequences that end earlier, as many batches one after another as
there are requests, slots given back and used again, limits."""
import pytest

from kidi_b200 import ErrorCode, KidiError
from kidi_b200.engine.generate import GenerationOptions, GenerationStats, generate
from kidi_b200.engine.search import SequenceState, plan_batches


class FakeBackend:
    """A model whose next token is (sum of the sequence's tokens) mod vocabulary."""

    def __init__(self, vocab_size=50, max_positions=64, token_budget=256, page=16, max_slots=8):
        self.vocab_size, self.max_positions = vocab_size, max_positions
        self.token_budget, self.page, self.max_slots = token_budget, page, max_slots
        self.free = list(range(max_slots - 1, -1, -1))
        self.sequences = {}
        self.log = []
        self.peak_live = 0
        self.acquired = []
        self.read_upto = {}

    def acquire(self):
        slot = self.free.pop()
        self.sequences[slot] = []
        self.acquired.append(slot)
        self.peak_live = max(self.peak_live, len(self.sequences))
        return slot

    def release(self, slot):
        assert slot in self.sequences, "a slot is released twice"
        del self.sequences[slot]
        self.free.append(slot)

    def _next(self, slot):
        return sum(self.sequences[slot]) % self.vocab_size

    def prefill(self, slots, chunks, select, temperature, keys, steps):
        self.log.append(("prefill", [len(chunk) for chunk in chunks], list(select)))
        for slot, chunk in zip(slots, chunks):
            self.sequences[slot].extend(chunk)
        return [self._next(slot) for slot, chosen in zip(slots, select) if chosen]

    def open_decode(self, slots, tokens, temperature, keys, steps, longest):
        backend = self
        self.log.append(("open", len(slots)))

        class Session:
            """Steps run when they are submitted (as on a device); a step is fed with the
            tokens of the step before it."""

            def __init__(self):
                self.tokens = list(tokens)
                self.results = []

            def submit(self):
                for slot, token in zip(slots, self.tokens):
                    assert slot in backend.sequences, "a step ran for a sequence whose slot was given back"
                    backend.sequences[slot].append(token)
                self.tokens = [backend._next(slot) for slot in slots]
                backend.log.append(("decode", len(slots)))
                self.results.append(list(self.tokens))
                assert len(self.results) - backend.read_upto.get(id(self), 0) <= 2, "more than one step ahead"
                return len(self.results) - 1

            def read(self, ticket):
                backend.read_upto[id(self)] = max(backend.read_upto.get(id(self), 0), ticket + 1)
                return list(self.results[ticket])

        return Session()


def expected(prompt, limit, stops, vocab=50):
    tokens, out = list(prompt), []
    for _ in range(limit):
        token = sum(tokens) % vocab
        if token in stops:
            return out, "stop"
        out.append(token)
        tokens.append(token)
    return out, "length"


def test_sequence_state_follows_the_greedy_bookkeeping():
    state = SequenceState(vocab_size=10, max_new_tokens=3, stop_ids=[9], ignore_eos=False)
    state.accept(4)
    state.accept(9)                       # a stop token ends the sequence and is not appended
    assert state.finished and state.result().token_ids == [4] and state.result().finish_reason == "stop"
    assert state.result().decoder_steps == 2 and not state.result().truncated
    with pytest.raises(KidiError):
        state.accept(1)                   # already finished
    state = SequenceState(10, 2, [9], ignore_eos=True)
    state.accept(9)
    state.accept(9)                       # --ignore-eos keeps end tokens and runs to the limit
    assert state.result().token_ids == [9, 9] and state.result().finish_reason == "length"
    state = SequenceState(10, 2, [9], False)
    state.accept(1)
    state.accept(2)
    assert state.finished and state.result().truncated
    with pytest.raises(KidiError) as caught:
        SequenceState(10, 5, [], False).accept(-1)   # no valid score
    assert caught.value.code == ErrorCode.RUNTIME


def test_unequal_prompts_stop_tokens_and_early_finish():
    backend = FakeBackend()
    prompts = [[1, 2, 3], [7], [4, 4, 4, 4, 4, 4, 4], [9, 9]]
    stops = [12, 28]
    options = GenerationOptions(max_new_tokens=6, max_active=4)
    stats = GenerationStats()
    results = generate(backend, prompts, options, stop_ids=stops, stats=stats)
    for prompt, result in zip(prompts, results):
        tokens, reason = expected(prompt, 6, stops)
        assert result.token_ids == tokens and result.finish_reason == reason
    assert {r.finish_reason for r in results} == {"stop", "length"}
    # One step for all four prompts, then fewer and fewer live rows.
    assert backend.log[0] == ("prefill", [3, 1, 7, 2], [True] * 4)
    live_counts = [entry[1] for entry in backend.log if entry[0] == "decode"]
    assert live_counts == sorted(live_counts, reverse=True) and live_counts[0] <= 4 and live_counts[-1] >= 1
    assert not backend.sequences and sorted(backend.free) == list(range(8))
    assert stats.prompt_tokens == 13 and stats.generated_tokens == sum(len(r.token_ids) for r in results)
    assert stats.batches == 1


def test_decoding_runs_one_step_ahead_and_a_stop_token_costs_nothing():
    """The loop submits step n+1 before it reads step n. When a stop token ends a sequence in
    step n, the step that ran ahead is kept for the others, and no step is submitted ahead
    when a sequence is about to reach its limit (its slot's room ends there)."""
    backend = FakeBackend()
    prompts = [[1, 2, 3], [7], [4, 4, 4, 4, 4, 4, 4], [9, 9]]
    stops = [12, 28]
    results = generate(backend, prompts, GenerationOptions(max_new_tokens=6, max_active=4), stop_ids=stops)
    for prompt, result in zip(prompts, results):
        tokens, reason = expected(prompt, 6, stops)
        assert result.token_ids == tokens and result.finish_reason == reason
        assert result.decoder_steps == len(tokens) + (reason == "stop")
    # A sequence never holds more tokens than its prompt and its limit allow (checked per step by
    # the fake session: a step for a released slot fails), and with limits alone no step is wasted:
    backend = FakeBackend()
    stats = GenerationStats()
    generate(backend, [[1], [2, 3]], GenerationOptions(max_new_tokens=5, ignore_eos=True), stats=stats)
    assert stats.decode_steps == 4 and [e for e in backend.log if e[0] == "decode"] == [("decode", 2)] * 4


def test_a_captured_step_is_kept_per_launch_signature(monkeypatch):
    """The engine's backend keeps one captured decode session per (batch bucket, launch
    signature): a later call whose longest sequence changes the model's launch choices gets a
    capture of its own, an equal one replays the first, and the number kept is bounded."""
    from kidi_b200.engine import decode_graph, generate as loop

    made = []

    class FakeSession:
        def __init__(self, engine, capacity, sampler, longest):
            self.capacity, self.longest = capacity, longest
            made.append((capacity, longest))

        def load(self, *arguments):
            pass

    class FakeModel:
        def launch_signature(self, rows, longest):
            return (rows, -(-longest // 1000))      # the choice changes every 1,000 tokens

    class FakeEngine:
        vocab_size = 10
        model = FakeModel()

        class spec:
            max_positions = 100000

        class cache:
            max_tokens, page_size, n_slots = 1 << 20, 64, 64

    monkeypatch.setattr(decode_graph, "DecodeSession", FakeSession)
    backend = loop.EngineBackend(FakeEngine(), sampler=None)
    open_for = lambda rows, longest: backend.open_decode(list(range(rows)), [0] * rows, [0.0] * rows, list(range(rows)),
                                                         [1] * rows, longest)
    short = open_for(3, 300)
    assert open_for(4, 900) is short and made == [(4, 300)]          # same bucket, same choices
    long = open_for(3, 5000)
    assert long is not short and made[-1] == (4, 5000)               # other choices: a capture of its own
    assert open_for(3, 400) is short
    for longest in range(10000, 10000 + 1000 * loop.MAX_KEPT_SESSIONS, 1000):
        open_for(3, longest)
    assert len(backend._sessions) == loop.MAX_KEPT_SESSIONS
    assert open_for(3, 300) is not short                             # the least recently used was dropped


def test_batches_follow_one_another_and_reuse_slots():
    backend = FakeBackend(max_slots=3)
    prompts = [[i + 1, i + 2] for i in range(8)]
    results = generate(backend, prompts, GenerationOptions(max_new_tokens=4, max_active=3, ignore_eos=True))
    assert [r.token_ids for r in results] == [expected(p, 4, [])[0] for p in prompts]
    assert backend.peak_live == 3
    assert [entry[1] for entry in backend.log if entry[0] == "prefill"] == [[2, 2, 2], [2, 2, 2], [2, 2]]
    assert set(backend.acquired) == {0, 1, 2} and len(backend.acquired) == 8     # the same slots again
    assert not backend.sequences


def test_the_token_budget_limits_a_batch():
    # Each request may come to hold 10 + 22 - 1 = 31 tokens -> 32 with pages of 16; 100 tokens hold three.
    batches = plan_batches([10] * 7, [22] * 7, token_budget=100, page=16, max_active=8, max_positions=64)
    assert batches == [(0, 3), (3, 6), (6, 7)]
    with pytest.raises(KidiError):
        plan_batches([10], [200], token_budget=100, page=16, max_active=8, max_positions=512)
    with pytest.raises(KidiError):
        plan_batches([60], [10], token_budget=1000, page=16, max_active=8, max_positions=64)


def test_limits_and_per_request_max_tokens():
    backend = FakeBackend()
    results = generate(backend, [[1], [2], [3]], GenerationOptions(max_new_tokens=5, ignore_eos=True),
                       max_tokens=[None, 2, 7])
    assert [len(r.token_ids) for r in results] == [5, 2, 7]
    with pytest.raises(KidiError) as caught:          # prompt and generation must fit the context
        generate(backend, [[1] * 60], GenerationOptions(max_new_tokens=10))
    assert caught.value.code == ErrorCode.INVALID_ARGUMENT
    with pytest.raises(KidiError):
        generate(backend, [[]], GenerationOptions())
    with pytest.raises(KidiError):
        generate(backend, [[50]], GenerationOptions())  # outside the vocabulary
    # Without an explicit limit a request gets what the context leaves (the default is larger).
    results = generate(backend, [[1] * 60], GenerationOptions(ignore_eos=True, context_size=64))
    assert len(results[0].token_ids) == 4
    assert not backend.sequences


def test_chunked_prompts_select_only_at_the_end():
    backend = FakeBackend()
    prompts = [[1] * 10, [2] * 3]
    results = generate(backend, prompts, GenerationOptions(max_new_tokens=2, prefill_chunk_size=4, ignore_eos=True))
    assert [entry for entry in backend.log if entry[0] == "prefill"] == [
        ("prefill", [4, 3], [False, True]), ("prefill", [4], [False]), ("prefill", [2], [True])]
    assert [r.token_ids for r in results] == [expected(p, 2, [])[0] for p in prompts]


def test_a_failure_gives_the_slots_back():
    backend = FakeBackend()

    def broken(*args, **kwargs):
        raise RuntimeError("device fault")

    backend.open_decode = broken
    with pytest.raises(RuntimeError):
        generate(backend, [[1], [2]], GenerationOptions(max_new_tokens=3, ignore_eos=True))
    assert not backend.sequences and len(backend.free) == 8
