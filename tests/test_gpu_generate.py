"""Generation on the GPU: greedy through the Python entry point and the command line,
temperature sampling with a seed, decode steps replayed as a graph against plain
steps, batches that follow one another."""
import json
import os

import numpy as np
import pytest

import plain_model

pytestmark = pytest.mark.gpu


def load(folder, dtype, **options):
    from kidi_b200 import Engine
    return Engine.load(folder, dtype=dtype, **options)


def check_teacher_forced(config, tensors, prompt, tokens, error, stops=()):
    """Every generated token is the plain model's best next token given the tokens before it
    (whole sequences, no cache), unless the plain model's two best logits lie closer together
    than `error` times the largest logit (the bound on the engine's bfloat16 difference): then
    either of those near-best tokens may have been chosen."""
    if not tokens:
        return 0
    logits = plain_model.forward(config, tensors, list(prompt) + list(tokens))[len(prompt) - 1:-1].float().numpy()
    close_calls = 0
    for position, token in enumerate(tokens):
        row = logits[position]
        best, second = np.sort(row)[-1], np.sort(row)[-2]
        bound = error * max(1.0, float(np.abs(row).max()))
        if best - second >= bound:
            assert token == int(np.argmax(row)), (prompt, tokens, position, float(best - second), bound)
        else:
            close_calls += 1
            assert row[token] >= best - bound, (prompt, tokens, position)
        assert token not in stops
    return close_calls


@pytest.mark.parametrize("use_graph", [True, False])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c"])
def test_greedy_generation_matches_the_plain_model_in_32_bit(model_folders, name, use_graph):
    config, tensors = plain_model.read_model_folder(model_folders[name])
    generator = np.random.default_rng(4)
    lengths = [5, 9, 13, 1, 30, 64, 2]
    prompts = [generator.integers(0, config["vocab_size"], size=n).tolist() for n in lengths]
    engine = load(model_folders[name], "float32", max_tokens=1024)
    found = engine.generate(prompts, max_new_tokens=8, ignore_eos=True, max_active=3, use_graph=use_graph)
    for prompt, tokens in zip(prompts, found):
        assert tokens == plain_model.generate(config, tensors, prompt, 8)
    engine.cache.check()
    assert not engine.cache.slots.held


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_d", "tiny_e"])
def test_greedy_generation_in_bfloat16(model_folders, name):
    config, tensors = plain_model.read_model_folder(model_folders[name])
    generator = np.random.default_rng(5)
    # Head widths 64 and 128 (tiny_d, tiny_e) take the tensor-memory prompt kernel and the
    # page-copy decode kernel: prompts longer than one of their tiles.
    lengths = [3, 17, 40, 8] if name in ("tiny_a", "tiny_b") else [3, 140, 200, 64]
    prompts = [generator.integers(0, config["vocab_size"], size=n).tolist() for n in lengths]
    engine = load(model_folders[name], "bfloat16", max_tokens=1024)
    found = engine.generate(prompts, max_new_tokens=12, ignore_eos=True)
    eager = engine.generate(prompts, max_new_tokens=12, ignore_eos=True, use_graph=False)
    from test_gpu_replay import BF16_TOLERANCES
    error = BF16_TOLERANCES[name][0]          # three times the measured bfloat16 difference
    close_calls = 0
    for prompt, tokens in zip(prompts, found):
        assert len(tokens) == 12
        close_calls += check_teacher_forced(config, tensors, prompt, tokens, error)
    for prompt, tokens in zip(prompts, eager):
        check_teacher_forced(config, tensors, prompt, tokens, error)
    assert close_calls <= len(prompts) * 12 // 4, "too many tokens are decided within the rounding error to test much"


def test_a_longer_call_gets_a_capture_of_its_own(model_folders):
    """The captured decode step freezes how attention splits a sequence's keys, chosen from the
    longest sequence the call may come to hold. A second call with much longer sequences must
    not replay the first call's graph: it captures one fitted to its own length, and both give
    the plain model's tokens."""
    config, tensors = plain_model.read_model_folder(model_folders["tiny_e"])
    generator = np.random.default_rng(8)
    engine = load(model_folders["tiny_e"], "float32", max_tokens=2048)
    bf16 = load(model_folders["tiny_e"], "bfloat16", max_tokens=2048)
    short = [generator.integers(0, config["vocab_size"], size=n).tolist() for n in (5, 9)]
    long = [generator.integers(0, config["vocab_size"], size=n).tolist() for n in (300, 340)]
    for prompts in (short, long, short):
        found = engine.generate(prompts, max_new_tokens=6, ignore_eos=True)
        assert found == [plain_model.generate(config, tensors, prompt, 6) for prompt in prompts]
        assert bf16.generate(prompts, max_new_tokens=6, ignore_eos=True) == \
            bf16.generate(prompts, max_new_tokens=6, ignore_eos=True, use_graph=False)
    sessions = next(iter(bf16._backends.values()))._sessions
    signatures = [key[1] for key in sessions]
    assert len(sessions) == 2 and signatures[0] != signatures[1], "the longer call replayed the shorter call's capture"
    assert all(key[0] == 2 for key in sessions)                    # one batch bucket, two launch signatures
    assert len(next(iter(engine._backends.values()))._sessions) == 1   # the 32-bit kernels choose nothing by length


def test_stop_tokens_end_a_sequence_early(model_folders):
    """A stop token chosen from what the model really generates: the sequence ends there,
    the token is not returned, and the others go on."""
    config, tensors = plain_model.read_model_folder(model_folders["tiny_b"])
    prompts = [[5, 6, 7], [100, 200, 300, 4], [42]]
    free = [plain_model.generate(config, tensors, prompt, 10) for prompt in prompts]
    stop = free[1][3]
    engine = load(model_folders["tiny_b"], "float32")
    found = engine.generate(prompts, max_new_tokens=10, stop_ids=[stop], detailed=True)
    for prompt, result in zip(prompts, found):
        expected = plain_model.generate(config, tensors, prompt, 10, stop_ids=[stop, 3, 11])
        assert result.token_ids == expected
        assert result.finish_reason == ("length" if len(expected) == 10 else "stop")
    assert len(found[1].token_ids) <= 3 and found[1].decoder_steps == len(found[1].token_ids) + 1
    ignoring = engine.generate(prompts, max_new_tokens=10, stop_ids=[stop], ignore_eos=True)
    assert ignoring == free


def test_temperature_sampling_is_seeded_and_independent_of_the_batch(model_folders):
    config, tensors = plain_model.read_model_folder(model_folders["tiny_b"])
    generator = np.random.default_rng(6)
    prompts = [generator.integers(0, 389, size=n).tolist() for n in [1, 7, 17, 31]]
    engine = load(model_folders["tiny_b"], "float32")
    first = engine.generate(prompts, max_new_tokens=12, temperature=0.8, seed=11, ignore_eos=True, max_active=4)
    again = engine.generate(prompts, max_new_tokens=12, temperature=0.8, seed=11, ignore_eos=True, max_active=4)
    other = engine.generate(prompts, max_new_tokens=12, temperature=0.8, seed=12, ignore_eos=True, max_active=4)
    alone = engine.generate(prompts, max_new_tokens=12, temperature=0.8, seed=11, ignore_eos=True, max_active=1)
    assert first == again and first != other
    assert first == alone                               # a sequence draws the same tokens in any batch
    assert first != engine.generate(prompts, max_new_tokens=12, ignore_eos=True)
    for key, (prompt, tokens) in enumerate(zip(prompts, first)):
        assert tokens == plain_model.generate(config, tensors, prompt, 12, temperature=0.8, seed=11, key=key)


def test_many_requests_in_batches_one_after_another(model_folders):
    config, tensors = plain_model.read_model_folder(model_folders["tiny_a"])
    generator = np.random.default_rng(7)
    prompts = [generator.integers(0, 256, size=int(n)).tolist() for n in generator.integers(1, 60, size=11)]
    engine = load(model_folders["tiny_a"], "float32", max_tokens=4 * 128)
    from kidi_b200.engine.generate import GenerationStats
    stats = GenerationStats()
    found = engine.generate(prompts, max_new_tokens=5, max_active=4, stats=stats, detailed=True)
    assert stats.batches >= 3 and stats.prompt_tokens == sum(len(p) for p in prompts)
    for prompt, result in zip(prompts, found):
        assert result.token_ids == plain_model.generate(config, tensors, prompt, 5, stop_ids=[7])
    engine.cache.check()
    assert not engine.cache.slots.held


def test_chunked_prompts_give_the_same_tokens(model_folders):
    config, tensors = plain_model.read_model_folder(model_folders["tiny_c"])
    generator = np.random.default_rng(8)
    prompts = [generator.integers(0, 301, size=n).tolist() for n in [150, 33, 90]]
    engine = load(model_folders["tiny_c"], "float32", max_tokens=1024)
    whole = engine.generate(prompts, max_new_tokens=4, ignore_eos=True)
    chunked = engine.generate(prompts, max_new_tokens=4, ignore_eos=True, prefill_chunk_size=32)
    assert whole == chunked == [plain_model.generate(config, tensors, p, 4) for p in prompts]


def test_command_line_generate(model_folders, tmp_path):
    import kidi_b200
    config, tensors = plain_model.read_model_folder(model_folders["tiny_a"])
    requests = [{"id": "x", "token_ids": [1, 2, 3, 4]}, {"token_ids": [9], "max_tokens": 3}, {"id": 5, "token_ids": [200, 100]}]
    source, sink = tmp_path / "in.jsonl", tmp_path / "out.jsonl"
    source.write_text("".join(json.dumps(request) + "\n" for request in requests))
    code = kidi_b200.main(["generate", "-m", model_folders["tiny_a"], "-i", str(source), "-o", str(sink),
                           "--max-new-tokens", "6", "--precision", "fp32", "--ignore-eos", "--profile",
                           "--cache-tokens", "512"])
    assert code == 0
    records = [json.loads(line) for line in sink.read_text().splitlines()]
    assert [record["id"] for record in records] == ["x", None, 5]
    assert [record["request_id"] for record in records] == [0, 1, 2]
    for request, record in zip(requests, records):
        limit = request.get("max_tokens", 6)
        assert record["token_ids"] == plain_model.generate(config, tensors, request["token_ids"], limit)
        assert record["decoder_steps"] == limit and record["finish"] == "length"
    source.write_text(json.dumps({"messages": []}) + "\n")
    assert kidi_b200.main(["generate", "-m", model_folders["tiny_a"], "-i", str(source), "-o", str(sink)]) == 1


def test_smoke_entry():
    import importlib.util
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("graft_entry", os.path.join(root, "__graft_entry__.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    module.smoke()
