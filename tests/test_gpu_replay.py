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
import torch

import replay_helpers as rh
from tiny_configs import ALL

pytestmark = pytest.mark.gpu

# 32-bit: both sides round at 2^-24 per operation; a few hundred operations deep.
FP32_TOLERANCE = 2e-5
# bfloat16: unit roundoff 2^-9 at about eight rounding points per layer, adding like a
# random walk, on logits of magnitude one.
BF16_TOLERANCE = 4e-2

LENGTHS = {
    "tiny_a": [1, 5, 33, 64, 65, 97, 128],
    "tiny_b": [1, 7, 17, 31, 66, 129, 200, 256],
    "tiny_c": [2, 40, 71, 141, 250, 320],
    "tiny_d": [3, 127, 128, 129, 300, 420],
    "tiny_e": [1, 130, 257, 384],
}


def tolerance(dtype):
    return FP32_TOLERANCE if dtype == "float32" else BF16_TOLERANCE


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
def test_whole_requests(model_folders, references, name, dtype):
    requests, expected = references[name]
    engine = make_engine(model_folders[name], dtype)
    rh.assert_matches(rh.run_whole(engine, requests), expected, tolerance(dtype), f"{name} {dtype} whole")
    engine.cache.check()
    assert not engine.cache.slots.held


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ALL))
def test_last_tokens_one_by_one(model_folders, references, name, dtype):
    requests, expected = references[name]
    engine = make_engine(model_folders[name], dtype)
    rh.assert_matches(rh.run_tail_decoded(engine, requests, 32), expected, tolerance(dtype),
                      f"{name} {dtype} last 32 one by one")
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ALL))
def test_unequal_batches_with_slot_reuse(model_folders, references, name, dtype):
    requests, expected = references[name]
    # A budget that holds one batch only, so that the next batch gets the same slots and pages.
    budget = sum(-(-length // 64) * 64 for length in sorted(LENGTHS[name])[-3:])
    engine = make_engine(model_folders[name], dtype, max_tokens=budget)
    found = rh.run_batches(engine, requests, batch_size=3, prompt_fraction=0.4)
    rh.assert_matches(found, expected, tolerance(dtype), f"{name} {dtype} batches of 3")
    engine.cache.check()
    assert not engine.cache.slots.held
    # The same requests again, in another grouping, on the used cache.
    found = rh.run_batches(engine, dict(reversed(list(requests.items()))), batch_size=2, prompt_fraction=0.8)
    rh.assert_matches(found, expected, tolerance(dtype), f"{name} {dtype} batches of 2, reversed")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ALL))
def test_prompts_in_chunks(model_folders, references, name, dtype):
    """Prompts fed 100 tokens at a time, two requests a batch: steps of several tokens that
    continue what the cache holds (pages, rings and the tensor-memory attention kernel's
    reading from the cache all meet a chunk boundary inside a page)."""
    requests, expected = references[name]
    engine = make_engine(model_folders[name], dtype)
    rh.assert_matches(rh.run_chunked(engine, requests, chunk=100), expected, tolerance(dtype),
                      f"{name} {dtype} in chunks of 100")
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
    rh.assert_matches(rh.run_tail_decoded(engine, requests, tail=64), expected, tolerance(dtype), "first tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model_folders, dtype):
    """One token a step from position 1 to the positional capacity: every page boundary
    and the wrap of the windowed ring are crossed while decoding."""
    name = "tiny_c"
    requests = rh.random_requests(ALL[name]["vocab_size"], [320, 300], seed=9)
    expected = rh.plain_logits(model_folders[name], requests)
    engine = make_engine(model_folders[name], dtype)
    rh.assert_matches(rh.run_batches(engine, requests, batch_size=2, prompt_fraction=0.0), expected,
                      tolerance(dtype), f"long decoding {dtype}")


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
    tol = tolerance(dtype)
    first = read(0)
    assert first.shape[0] == 40
    assert rh.relative_error(first[:38], expected["r0"][:38]) <= tol
    assert rh.relative_error(first[38:], expected["r1"][[0, 59]]) <= tol
    assert rh.relative_error(read(1), np.stack([expected["r0"][38], expected["r1"][60]])) <= tol
    assert rh.relative_error(read(10), expected["r1"][69:70]) <= tol
    assert rh.relative_error(read(11), expected["r2"][-1:]) <= tol
