"""A two-layer model with the layer sizes of the benchmark (hidden 4096, 32 query heads over
8 key/value heads of width 128, intermediate 12288, a vocabulary of 151,936) against the plain
implementation, in steps of 1, 8, 12, 16, 24 and 64 sequences, through `Engine.step` and
through the replayed decode graph, twice in a row so that slots and pages are used again.

Which kernel a product or an attention step takes depends on thresholds that only these sizes
reach (the weight-streaming product up to 8 rows, the tcgen05 product with the fused gate
from 9 to 16 rows of a tall weight, the vendor library elsewhere, the two-stage argmax, the
ring form and the cluster merge of decode attention). Every case asserts which kernels ran,
so that a change of a threshold cannot quietly take a branch out of the test."""
import numpy as np
import pytest
import torch

import plain_model

pytestmark = pytest.mark.gpu

SHAPE = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu",
    "num_hidden_layers": 2, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 4096,
}
SEQUENCES = 64
DECODED = 3            # the last tokens of every sequence come one by one
LONG = 200             # the first sequence is this long: several pages, so that its keys are split
# Relative to a sequence's largest logit (about 6). Measured on a B200 over all batch sizes:
# 6.4e-6 in 32-bit (products of 4096 to 12288 terms), 1.1e-2 to 1.3e-2 in bfloat16; the bounds
# are three and two times that. Every case records what it measures (`record_property`).
FP32_TOLERANCE = 2e-5
BF16_TOLERANCE = 2.5e-2


@pytest.fixture(scope="module")
def shape_model():
    """Weights drawn on the device (bfloat16), the same tensors on the host in 32-bit for the
    plain model, and the plain logits of every sequence at its last DECODED + 1 positions."""
    from kidi_b200.engine.model import declared_parameters
    from kidi_b200.registry import spec_from_config
    from kidi_b200.weights.random_init import checkpoint_tensors
    device = torch.device("cuda:0")
    params = declared_parameters(spec_from_config(SHAPE)[2])
    tensors = dict(checkpoint_tensors(params, seed=3, dtype=torch.bfloat16, device=device))
    host = {name: tensor.float().cpu() for name, tensor in tensors.items()}
    generator = np.random.default_rng(17)
    lengths = [LONG] + [int(n) for n in generator.integers(DECODED + 2, 24, size=SEQUENCES - 1)]
    sequences = [generator.integers(0, SHAPE["vocab_size"], size=n).tolist() for n in lengths]
    expected = []
    torch.set_num_threads(max(1, torch.get_num_threads()))
    for tokens in sequences:
        expected.append(plain_tail_logits(host, tokens, DECODED + 1))
    del host
    return tensors, sequences, expected


def plain_tail_logits(tensors, tokens, tail):
    """The plain model's logits at the last `tail` positions (its parts, called in its order; the
    head only where it is wanted: a full-width head over 200 positions is a quarter of a TFLOP)."""
    config = SHAPE
    cos, sin = plain_model.rotary_tables(len(tokens), config["head_dim"], plain_model.rope_theta(config))
    hidden = plain_model.embed(tokens, tensors["model.embed_tokens.weight"])
    for layer in range(config["num_hidden_layers"]):
        hidden = plain_model.block(hidden, tensors, layer, config, cos, sin, None)
    hidden = plain_model.rms_norm(hidden[-tail:], tensors["model.norm.weight"], config["rms_norm_eps"])
    return (hidden @ tensors["lm_head.weight"].T).numpy()


_engines = {}


def engine_of(shape_model, dtype):
    from kidi_b200 import Engine
    if dtype not in _engines:
        _engines.clear()   # one engine at a time: the 32-bit one holds 6.6 GB of weights
        torch.cuda.empty_cache()
        _engines[dtype] = Engine.from_config(SHAPE, dtype=dtype, tensors=shape_model[0], max_tokens=64 * 256,
                                             max_slots=64)
    return _engines[dtype]


def relative_error(found, expected):
    return float(np.abs(found - expected).max() / max(1.0, float(np.abs(expected).max())))


def run_steps(engine, sequences, use_graph):
    """Prompts (all but the last DECODED tokens) in one step, then DECODED single tokens; returns
    [sequence][DECODED + 1, vocab] logits and the names of the kernels of the last decode step."""
    from kidi_b200 import StepBatch
    from kidi_b200.engine.decode_graph import DecodeSession
    from kidi_b200.kernels import ops
    from kidi_b200.sampling.sampler import Sampler
    count = len(sequences)
    slots = [engine.acquire() for _ in sequences]
    try:
        heads = [len(tokens) - DECODED for tokens in sequences]
        logits = engine.step(StepBatch(slots, [tokens[:head] for tokens, head in zip(sequences, heads)], None))
        rows = [[logits[index].cpu().numpy()] for index in range(count)]
        names = []
        if use_graph:
            capacity = 1
            while capacity < count:
                capacity *= 2
            session = DecodeSession(engine, capacity, Sampler(0), longest=max(len(tokens) for tokens in sequences))
            session.load(slots, [tokens[head] for tokens, head in zip(sequences, heads)], [0.0] * count,
                         list(range(count)), [1] * count)
        for step in range(DECODED):
            fed = [tokens[head + step] for tokens, head in zip(sequences, heads)]
            if use_graph:
                with ops.record_launches() as names:        # the first step captures: its launches are the graph's
                    session.step(fed)
                logits = session.logits[:count]
            else:
                with ops.record_launches() as names:
                    logits = engine.step(StepBatch(slots, [[token] for token in fed], None))
            for index in range(count):
                rows[index].append(logits[index].cpu().numpy())
            if step == 0:
                first_names = list(names)
        return [np.stack(found) for found in rows], first_names
    finally:
        for slot in slots:
            engine.release(slot)
        engine.cache.check()


# What each batch size has to run in bfloat16 (substrings of the recorded names): the products
# of a layer are qkv, o, gate/up, down; the head follows.
EXPECTED_KERNELS = {
    1: ["gemm_skinny[row factors]", "gemm_skinny[into the residual]", "gemm_silu_gate[skinny]", "attention_decode[cluster]"],
    8: ["gemm_skinny[row factors]", "gemm_skinny[into the residual]", "gemm_silu_gate[skinny]", "attention_decode[cluster]"],
    12: ["library_mm", "gemm_silu_gate[tcgen05]", "gemm_tcgen05", "attention_decode[cluster]"],
    16: ["library_mm", "gemm_silu_gate[tcgen05]", "gemm_tcgen05", "attention_decode[cluster]"],
    24: ["library_mm", "silu_gate", "gemm_tcgen05", "attention_decode[cluster]"],        # the head: tcgen05
    32: ["library_mm", "silu_gate", "gemm_tcgen05", "attention_decode[one block]"],     # 24 sequences padded by the graph
    64: ["library_mm", "silu_gate", "gemm_tcgen05", "attention_decode[ring]"],
}


@pytest.mark.parametrize("use_graph", [False, True], ids=["step", "graph"])
@pytest.mark.parametrize("count", [1, 8, 12, 16, 24, 64])
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_benchmark_sizes_against_the_plain_model(shape_model, record_property, dtype, count, use_graph):
    _, sequences, expected = shape_model
    engine = engine_of(shape_model, dtype)
    tolerance = BF16_TOLERANCE if dtype == "bfloat16" else FP32_TOLERANCE
    worst = 0.0
    for turn in range(2):                                  # the second turn runs on used slots and pages
        found, names = run_steps(engine, sequences[:count], use_graph)
        for index in range(count):
            assert np.isfinite(found[index]).all()
            error = relative_error(found[index], expected[index])
            worst = max(worst, error)
            assert error <= tolerance, (f"{dtype}, {count} sequences, turn {turn}: sequence {index} of "
                                        f"{len(sequences[index])} tokens differs by {error:.3e}")
    record_property("max_error", worst)                    # in the junit report: what the tolerance is fitted to
    if dtype == "bfloat16":
        ran = count if not use_graph else 1 << (count - 1).bit_length()   # the graph pads to a power of two
        for wanted in EXPECTED_KERNELS[ran]:
            assert any(wanted in name for name in names), f"{wanted} did not run at {ran} rows: {sorted(set(names))}"
        assert any("argmax" in name or "sample" in name for name in names) or not use_graph
        if ran <= 8:
            # The norms between the products have no kernel of their own: only the first layer's input
            # norm and the final norm are launched (the graph's list holds its warm-up run as well).
            assert names.count("add_rmsnorm") == (4 if use_graph else 2), names
            assert "library_mm" not in names
    else:
        assert all("library" not in name and "tcgen05" not in name and "skinny" not in name for name in names), \
            f"the 32-bit engine left its 32-bit kernels: {sorted(set(names))}"
    engine.check_device_errors()


@pytest.mark.parametrize("form,count,setting", [
    ("merge in the last block", 1, {"cluster": 0}),
    ("combine kernel", 24, {"cluster": 0, "splits": "4"}),
    ("one block", 8, {"splits": "1"}),
])
def test_other_forms_of_decode_attention_whole_model(shape_model, monkeypatch, form, count, setting):
    """The forms of decode attention that the launcher takes at other lengths and batch sizes
    (splits merged through a workspace by the last block or by a second kernel, no splits),
    asked for here, in the whole model."""
    from kidi_b200.kernels import attention
    _, sequences, expected = shape_model
    if "cluster" in setting:
        monkeypatch.setattr(attention, "CLUSTER_SPLITS", setting["cluster"])
    if "splits" in setting:
        monkeypatch.setenv("KIDI_B200_DECODE_SPLITS", setting["splits"])
    engine = engine_of(shape_model, "bfloat16")
    found, names = run_steps(engine, sequences[:count], use_graph=False)
    assert any(f"attention_decode[{form}]" in name for name in names), sorted(set(names))
    for index in range(count):
        assert relative_error(found[index], expected[index]) <= BF16_TOLERANCE, (form, index)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_a_long_prompt_at_the_benchmark_sizes(shape_model, dtype):
    """A prompt of 1,100 tokens: from 1,024 rows on every product of the bfloat16 engine runs on this
    package's tcgen05 kernel in its compute-bound form (whole tiles, persistent blocks, TMA stores)
    and attention on the tcgen05 prompt kernel; no vendor-library product is left in the step."""
    from kidi_b200 import StepBatch
    from kidi_b200.kernels import ops
    tensors, _, _ = shape_model
    generator = np.random.default_rng(29)
    tokens = generator.integers(0, SHAPE["vocab_size"], size=1100).tolist()
    host = {name: tensor.float().cpu() for name, tensor in tensors.items()}
    expected = plain_tail_logits(host, tokens, 3)
    del host
    engine = engine_of(shape_model, dtype)
    slot = engine.acquire()
    try:
        with ops.record_launches() as names:
            first = engine.step(StepBatch([slot], [tokens[:-1]], [[len(tokens) - 3, len(tokens) - 2]])).cpu().numpy()
        last = engine.step(StepBatch([slot], [tokens[-1:]], None)).cpu().numpy()
    finally:
        engine.release(slot)
    found = np.concatenate([first, last])
    tolerance = BF16_TOLERANCE if dtype == "bfloat16" else FP32_TOLERANCE
    assert relative_error(found, expected) <= tolerance, relative_error(found, expected)
    if dtype == "bfloat16":
        assert names.count("gemm_tcgen05") == 4 * SHAPE["num_hidden_layers"] and "library_mm" not in names, sorted(set(names))
        assert "attention_prefill_tcgen05" in names
    engine.check_device_errors()
