"""The engine against the plain implementation under every way of cutting the work:
each request alone and whole; with the last 32 tokens one by one; in batches of unequal
lengths whose shorter requests end earlier, one batch after another so that slots are
used again; in 32-bit and in bfloat16."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import replay_helpers as rh
from tiny_configs import ALL

pytestmark = pytest.mark.gpu

# Differences are relative to a request's largest logit (6 to 12: the models' final norm is
# scaled so, see conftest.sharpen_logits). The bounds are three times what was measured on a
# B200 over all four ways of cutting (the largest difference, the root mean square over all
# logits); every test records what it measures (`record_property`, in the junit report).
# 32-bit: both sides round at 2^-24 per operation, a few hundred operations deep; measured
# 3.4e-7 to 1.2e-6.
FP32_TOLERANCE = 4e-6
# bfloat16 (unit roundoff 2^-9, about eight rounding points per layer, adding like a random
# walk): measured largest / root mean square per configuration:
#   tiny_a 2.6e-3 / 3.6e-4, tiny_b 7.3e-3 / 1.2e-3, tiny_c 6.9e-3 / 1.1e-3,
#   tiny_d 4.9e-3 / 8.6e-4, tiny_e 5.2e-3 / 8.6e-4.
BF16_TOLERANCES = {"tiny_a": (8e-3, 1.1e-3), "tiny_b": (2.2e-2, 3.5e-3), "tiny_c": (2.1e-2, 3.3e-3),
                   "tiny_d": (1.5e-2, 2.6e-3), "tiny_e": (1.6e-2, 2.6e-3)}
BF16_TOLERANCE = max(bound for bound, _ in BF16_TOLERANCES.values())

LENGTHS = {
    "tiny_a": [1, 5, 33, 64, 65, 97, 128],
    "tiny_b": [1, 7, 17, 31, 66, 129, 200, 256],
    "tiny_c": [2, 40, 71, 141, 250, 320],
    "tiny_d": [3, 127, 128, 129, 300, 420],
    "tiny_e": [1, 130, 257, 384],
}


def tolerance(dtype, name=None, rms=True):
    """The bound on the largest difference and, with `rms`, on the root mean square (fitted to the
    four cuts of the whole request set; tests of a few requests bound the largest difference only)."""
    if dtype == "float32":
        return FP32_TOLERANCE
    if name is None:
        return BF16_TOLERANCE
    return BF16_TOLERANCES[name] if rms else BF16_TOLERANCES[name][0]


def record(record_property, found, expected):
    record_property("max_error", rh.worst_error(found, expected))
    record_property("rms_error", rh.rms_error(found, expected))


@pytest.fixture(scope="module")
def references(model_folders):
    out = {}
    for name, folder in model_folders.items():
        config = ALL[name]
        requests = rh.random_requests(config["vocab_size"], LENGTHS[name], seed=11)
        out[name] = (requests, rh.plain_logits(folder, requests))
    return out


def make_engine(folder, dtype, max_tokens=2048):
    from kidi_b200 import Engine
    return Engine.load(folder, dtype=dtype, max_tokens=max_tokens)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ALL))
def test_whole_requests(model_folders, references, record_property, name, dtype):
    requests, expected = references[name]
    engine = make_engine(model_folders[name], dtype)
    found = rh.run_whole(engine, requests)
    record(record_property, found, expected)
    rh.assert_matches(found, expected, tolerance(dtype, name), f"{name} {dtype} whole")
    engine.cache.check()
    assert not engine.cache.slots.held


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ALL))
def test_last_tokens_one_by_one(model_folders, references, record_property, name, dtype):
    requests, expected = references[name]
    engine = make_engine(model_folders[name], dtype)
    found = rh.run_tail_decoded(engine, requests, 32)
    record(record_property, found, expected)
    rh.assert_matches(found, expected, tolerance(dtype, name), f"{name} {dtype} last 32 one by one")
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ALL))
def test_unequal_batches_with_slot_reuse(model_folders, references, record_property, name, dtype):
    requests, expected = references[name]
    # A budget that holds one batch only, so that the next batch gets the same slots and pages.
    budget = sum(-(-length // 64) * 64 for length in sorted(LENGTHS[name])[-3:])
    engine = make_engine(model_folders[name], dtype, max_tokens=budget)
    found = rh.run_batches(engine, requests, batch_size=3, prompt_fraction=0.4)
    record(record_property, found, expected)
    rh.assert_matches(found, expected, tolerance(dtype, name), f"{name} {dtype} batches of 3")
    engine.cache.check()
    assert not engine.cache.slots.held
    # The same requests again, in another grouping, on the used cache.
    found = rh.run_batches(engine, dict(reversed(list(requests.items()))), batch_size=2, prompt_fraction=0.8)
    rh.assert_matches(found, expected, tolerance(dtype, name), f"{name} {dtype} batches of 2, reversed")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ALL))
def test_prompts_in_chunks(model_folders, references, record_property, name, dtype):
    """Prompts fed 100 tokens at a time, two requests a batch: steps of several tokens that
    continue what the cache holds (pages, rings and the tensor-memory attention kernel's
    reading from the cache all meet a chunk boundary inside a page)."""
    requests, expected = references[name]
    engine = make_engine(model_folders[name], dtype)
    found = rh.run_chunked(engine, requests, chunk=100)
    record(record_property, found, expected)
    rh.assert_matches(found, expected, tolerance(dtype, name), f"{name} {dtype} in chunks of 100")
    engine.cache.check()
    assert not engine.cache.slots.held


@pytest.mark.parametrize("name", list(ALL))
def test_cuts_agree_in_32_bit(model_folders, references, name):
    """In 32-bit the logits of a position do not depend on the cut at all: the kernels
    accumulate in an order that depends on the position only."""
    requests, _ = references[name]
    engine = make_engine(model_folders[name], "float32")
    whole = rh.run_whole(engine, requests)
    tail = rh.run_tail_decoded(engine, requests, 32)
    batched = rh.run_batches(engine, requests, batch_size=4)
    for request in requests:
        assert np.array_equal(tail[request], whole[request]), request
        assert np.array_equal(batched[request], whole[request]), request


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(model_folders, dtype):
    """Positions 0, 1, 2: one token at a time from an empty cache."""
    name = "tiny_b"
    requests = rh.random_requests(ALL[name]["vocab_size"], [3, 2, 1], seed=5)
    expected = rh.plain_logits(model_folders[name], requests)
    engine = make_engine(model_folders[name], dtype)
    rh.assert_matches(rh.run_tail_decoded(engine, requests, tail=64), expected, tolerance(dtype, name, rms=False), "first tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model_folders, dtype):
    """One token a step from position 1 to the positional capacity: every page boundary
    and the wrap of the windowed ring are crossed while decoding."""
    name = "tiny_c"
    requests = rh.random_requests(ALL[name]["vocab_size"], [320, 300], seed=9)
    expected = rh.plain_logits(model_folders[name], requests)
    engine = make_engine(model_folders[name], dtype)
    rh.assert_matches(rh.run_batches(engine, requests, batch_size=2, prompt_fraction=0.0), expected,
                      tolerance(dtype, name, rms=False), f"long decoding {dtype}")


@pytest.mark.parametrize("ring", [False, True], ids=["pages", "ring"])
@pytest.mark.parametrize("name", ["tiny_d", "tiny_e"])
def test_a_page_that_is_used_again_carries_nothing_over(model_folders, references, monkeypatch, name, ring):
    """Head widths 64 and 128 copy whole 64-row pages: rows past a sequence's end are whatever
    the page held. A first request takes every page of a small cache; when it has ended, all
    keys and values are overwritten with NaN (a plain write through torch), as if that request
    had overflowed. The requests that then get its pages (whole, in chunks, token by token,
    in batches; decoding in the page-copying and in the ring form) must see none of it."""
    from kidi_b200 import StepBatch
    from kidi_b200.kernels import attention
    if ring:
        monkeypatch.setattr(attention, "DECODE_RING_ALWAYS", True)
    requests, expected = references[name]
    longest = max(len(tokens) for tokens in requests.values())
    budget = -(-longest // 64) * 64
    engine = make_engine(model_folders[name], "bfloat16", max_tokens=budget)
    slot = engine.acquire()
    engine.step(StepBatch([slot], [max(requests.values(), key=len)], None))
    assert all(group.pool.free_count == 0 for group in engine.cache.kv_groups if not group.ring_pages)
    engine.release(slot)
    for group in engine.cache.kv_groups:
        group.keys.fill_(float("nan"))
        group.values.fill_(float("nan"))
    tol = tolerance("bfloat16", name, rms=False)
    short = {name_: tokens for name_, tokens in requests.items() if len(tokens) <= budget // 2}
    rh.assert_matches(rh.run_whole(engine, requests), expected, tol, "whole, on poisoned pages")
    rh.assert_matches(rh.run_tail_decoded(engine, requests, 32), expected, tol, "last 32 one by one, on poisoned pages")
    rh.assert_matches(rh.run_chunked(engine, short, chunk=50, batch_size=1), {n: expected[n] for n in short}, tol,
                      "in chunks, on poisoned pages")
    engine.cache.check()


@pytest.mark.parametrize("name", list(ALL))
def test_the_bfloat16_comparison_notices_swapped_pages(model_folders, references, name):
    """A mutation that the comparison has to catch, or its tolerance is too wide: two sequences
    run their prompts together; then the first page of the one and the first page of the other
    change places in the block table of one group of layers (both are held pages of that
    group's pool, so nothing is read out of range), and both decode on. Without the swap the
    decoded logits match the plain model; with it they must not."""
    from kidi_b200 import StepBatch
    requests, expected = references[name]
    first, second = sorted(requests, key=lambda request: len(requests[request]))[-2:]
    tail = 16

    def decode_tails(swap: bool):
        engine = make_engine(model_folders[name], "bfloat16")
        slots = {request: engine.acquire() for request in (first, second)}
        heads = {request: len(requests[request]) - tail for request in slots}
        engine.step(StepBatch([slots[first], slots[second]], [requests[r][:heads[r]] for r in (first, second)], [[], []]))
        if swap:
            group = engine.cache.kv_groups[0]
            a, b = slots[first], slots[second]
            group.table_host[a, 0], group.table_host[b, 0] = group.table_host[b, 0], group.table_host[a, 0]
            group._dirty.update((a, b))
            engine.cache.flush_tables()
        rows = {request: [] for request in slots}
        for step in range(tail):
            logits = engine.step(StepBatch([slots[first], slots[second]],
                                           [[requests[r][heads[r] + step]] for r in (first, second)], None)).cpu().numpy()
            rows[first].append(logits[0])
            rows[second].append(logits[1])
        return {request: np.stack(found) for request, found in rows.items()}

    reference = {request: expected[request][-tail:] for request in (first, second)}
    bound = BF16_TOLERANCES[name][0]
    rh.assert_matches(decode_tails(swap=False), reference, bound, f"{name}: unswapped control")
    mutated = decode_tails(swap=True)
    for request in (first, second):
        assert rh.first_bad_position(mutated[request], reference[request], bound) is not None, \
            f"{name}: swapped cache pages of {request} stay within the bfloat16 tolerance"


@pytest.mark.parametrize("name", list(ALL))
def test_the_bfloat16_engine_against_the_32_bit_engine(model_folders, references, name):
    """The same cuts in both engines, compared with each other at the bfloat16 bound: the 32-bit
    engine shares its tables, cache and step function with the bfloat16 one and none of its
    product or attention kernels."""
    requests, _ = references[name]
    wide = make_engine(model_folders[name], "float32")
    narrow = make_engine(model_folders[name], "bfloat16")
    bound = tolerance("bfloat16", name)
    for what, run in (("whole", rh.run_whole), ("last 32 one by one", lambda e, r: rh.run_tail_decoded(e, r, 32)),
                      ("batches of 3", lambda e, r: rh.run_batches(e, r, batch_size=3, prompt_fraction=0.4)),
                      ("chunks of 100", lambda e, r: rh.run_chunked(e, r, chunk=100))):
        rh.assert_matches(run(narrow, requests), run(wide, requests), bound, f"{name} bfloat16 against 32-bit, {what}")


@pytest.mark.parametrize("name", ["tiny_b", "tiny_e"])
def test_folders_stored_in_32_bit_and_in_shards(model_folders, references, tmp_path, name):
    """The same weights stored as float32 (what the file holds is the bfloat16 values, widened),
    and spread over three shards behind model.safetensors.index.json: every engine reads them to
    the same logits. A bfloat16 engine keeps 32-bit matrices 32-bit and says so; asked to, it
    rounds them and then computes what it computes from the bfloat16 folder, bit for bit."""
    import shutil
    from kidi_b200 import Engine
    from kidi_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    requests, expected = references[name]
    requests = dict(list(requests.items())[:4])
    expected = {request: expected[request] for request in requests}
    source = SafetensorsFile(os.path.join(model_folders[name], "model.safetensors"))
    tensors = {tensor: source.tensor(tensor).clone() for tensor in source.names()}
    source.close()
    wide_folder, sharded_folder = tmp_path / "wide", tmp_path / "sharded"
    for folder in (wide_folder, sharded_folder):
        folder.mkdir()
        shutil.copy(os.path.join(model_folders[name], "config.json"), folder / "config.json")
    write_safetensors(str(wide_folder / "model.safetensors"), {n: t.float() for n, t in tensors.items()})
    names = sorted(tensors)
    weight_map = {}
    for index in range(3):
        file = f"model-{index + 1:05d}-of-00003.safetensors"
        members = names[index::3]
        write_safetensors(str(sharded_folder / file), {n: tensors[n] for n in members})
        weight_map.update({n: file for n in members})
    (sharded_folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))

    reference = rh.run_whole(make_engine(model_folders[name], "bfloat16"), requests)
    sharded = Engine.load(str(sharded_folder), dtype="bfloat16", max_tokens=2048)
    assert all(np.array_equal(found, reference[request]) for request, found in rh.run_whole(sharded, requests).items())
    wide32 = Engine.load(str(wide_folder), dtype="float32", max_tokens=2048)
    rh.assert_matches(rh.run_tail_decoded(wide32, requests, 32), expected, FP32_TOLERANCE, "float32 folder, 32-bit engine")
    with pytest.warns(UserWarning, match="32-bit kernel"):
        kept = Engine.load(str(wide_folder), dtype="bfloat16", max_tokens=2048)
    rh.assert_matches(rh.run_batches(kept, requests, batch_size=3), expected, tolerance("bfloat16", name, rms=False),
                      "float32 folder, bfloat16 engine with 32-bit weights")
    cast = Engine.load(str(wide_folder), dtype="bfloat16", max_tokens=2048, cast_weights=True)
    assert all(np.array_equal(found, reference[request]) for request, found in rh.run_whole(cast, requests).items())


def test_padding_changes_nothing(model_folders):
    """A request's logits are the same alone and beside a much longer neighbour."""
    name = "tiny_a"
    requests = rh.random_requests(ALL[name]["vocab_size"], [9, 120], seed=3)
    engine = make_engine(model_folders[name], "float32")
    alone = rh.run_whole(engine, {"r0": requests["r0"]})
    together = rh.run_batches(engine, requests, batch_size=2, prompt_fraction=1.0)
    assert np.array_equal(alone["r0"], together["r0"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_folders, tmp_path, dtype):
    """bin/trace_run end to end: a batch of two unequal requests, then a third request
    on the slots they gave back."""
    name = "tiny_b"
    requests = rh.random_requests(ALL[name]["vocab_size"], [40, 70, 50], seed=21)
    expected = rh.plain_logits(model_folders[name], requests)
    a, b, c = requests["r0"], requests["r1"], requests["r2"]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:38], "want": list(range(38))},
                                     {"id": "b", "tokens": b[:60], "want": [0, 59]}], "end": []}]
    for index in range(10):
        entries = [{"id": "b", "tokens": [b[60 + index]], "want": [0]}]
        if index < 2:
            entries.insert(0, {"id": "a", "tokens": [a[38 + index]], "want": [0]})
        steps.append({"step": 1 + index, "entries": entries,
                      "end": (["a"] if index == 1 else []) + (["b"] if index == 9 else [])})
    steps.append({"step": 11, "entries": [{"id": "c", "tokens": c, "want": [len(c) - 1]}], "end": ["c"]})
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    result = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", model_folders[name], "--dtype", dtype,
         "--out", str(out), "--max-tokens", "192"],
        input="\n".join(json.dumps(step) for step in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr
    assert result.stdout.split() == [word for step in steps for word in ("done", str(step["step"]))]
    vocab = ALL[name]["vocab_size"]
    read = lambda step: np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(-1, vocab)
    tol = tolerance(dtype, name, rms=False)
    first = read(0)
    assert first.shape[0] == 40
    assert rh.relative_error(first[:38], expected["r0"][:38]) <= tol
    assert rh.relative_error(first[38:], expected["r1"][[0, 59]]) <= tol
    assert rh.relative_error(read(1), np.stack([expected["r0"][38], expected["r1"][60]])) <= tol
    assert rh.relative_error(read(10), expected["r1"][69:70]) <= tol
    assert rh.relative_error(read(11), expected["r2"][-1:]) <= tol
