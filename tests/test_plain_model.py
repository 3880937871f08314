"""The plain implementation itself (no GPU): each part against an independent,
element-by-element restatement of its formula, and the invariants of the whole."""
import math

import numpy as np
import pytest
import torch

import plain_model
from kidi_b200 import write_random_model
from tiny_configs import ALL, TINY_B


def test_rms_norm_matches_the_closed_form():
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
    w = torch.tensor([1.0, 0.5, 2.0, 1.0])
    inv = 1.0 / math.sqrt(7.5 + 1e-6)   # mean of squares is 7.5, as in the reference's own test
    assert torch.allclose(plain_model.rms_norm(x, w, 1e-6), torch.tensor([[inv, inv, 6 * inv, 4 * inv]]), atol=1e-6)


def test_rotation_is_the_half_split_pairing():
    cos, sin = plain_model.rotary_tables(5, 4, 100.0)
    assert cos.shape == (5, 2) and float(cos[0, 0]) == 1.0 and float(sin[0, 1]) == 0.0
    assert abs(float(cos[3, 1]) - math.cos(3 * (1 / 100.0 ** 0.5))) < 1e-6
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]])
    out = plain_model.norm_then_rotate(x, torch.ones(4), 0.0, cos[2:3], sin[2:3])
    n = x[0, 0] / math.sqrt(7.5)
    c0, c1, s0, s1 = float(cos[2, 0]), float(cos[2, 1]), float(sin[2, 0]), float(sin[2, 1])
    want = [n[0] * c0 - n[2] * s0, n[1] * c1 - n[3] * s1, n[2] * c0 + n[0] * s0, n[3] * c1 + n[1] * s1]
    assert torch.allclose(out[0, 0], torch.tensor(want), atol=1e-6)


def test_attention_against_probabilities_by_hand():
    q = torch.tensor([[[1.0, 0.0]], [[0.0, 2.0]]])                  # two positions, one head
    k = torch.tensor([[[1.0, 0.0]], [[0.0, 1.0]]])
    v = torch.tensor([[[1.0, 10.0]], [[3.0, 30.0]]])
    out = plain_model.causal_attention(q, k, v)
    assert torch.allclose(out[0], torch.tensor([1.0, 10.0]))        # the first position sees itself only
    p = math.exp(2 / math.sqrt(2)) / (1 + math.exp(2 / math.sqrt(2)))
    assert torch.allclose(out[1], torch.tensor([1 - p + 3 * p, 10 * (1 - p) + 30 * p]), atol=1e-5)
    windowed = plain_model.causal_attention(q, k, v, window=1)      # a window of one: itself only
    assert torch.allclose(windowed[1], torch.tensor([3.0, 30.0]))


def test_grouped_heads_read_their_own_key_head():
    generator = torch.Generator().manual_seed(0)
    q, k, v = torch.randn(6, 4, 8, generator=generator), torch.randn(6, 2, 8, generator=generator), \
        torch.randn(6, 2, 8, generator=generator)
    out = plain_model.causal_attention(q, k, v).reshape(6, 4, 8)
    for head in range(4):
        alone = plain_model.causal_attention(q[:, head:head + 1], k[:, head // 2:head // 2 + 1],
                                             v[:, head // 2:head // 2 + 1])
        assert torch.allclose(out[:, head], alone.reshape(6, 8), atol=1e-6)


@pytest.mark.parametrize("name", list(ALL))
def test_the_model_is_causal_and_precision_is_in_hand(tmp_path, name):
    folder = write_random_model(ALL[name], str(tmp_path / name), seed=5)
    config, tensors = plain_model.read_model_folder(folder)
    tokens = np.random.default_rng(1).integers(0, config["vocab_size"], size=90).tolist()
    whole = plain_model.forward(config, tensors, tokens)
    assert whole.shape == (90, config["vocab_size"]) and torch.isfinite(whole).all()
    prefix = plain_model.forward(config, tensors, tokens[:40])
    assert torch.allclose(whole[:40], prefix, atol=2e-5)            # later tokens change nothing earlier
    double = plain_model.forward(config, tensors, tokens, dtype=torch.float64)
    assert float((whole.double() - double).abs().max()) < 2e-5


def test_the_window_matters(tmp_path):
    """With the window taken away the logits beyond it change: the configuration's window is used."""
    folder = write_random_model(TINY_B, str(tmp_path / "b"), seed=6)
    config, tensors = plain_model.read_model_folder(folder)
    tokens = list(range(1, 61))
    with_window = plain_model.forward(config, tensors, tokens)
    no_window = plain_model.forward(dict(config, layer_types=["full_attention"] * 3), tensors, tokens)
    assert torch.allclose(with_window[:24], no_window[:24], atol=1e-6)
    assert float((with_window[40:] - no_window[40:]).abs().max()) > 1e-4


def test_sampling_helpers():
    assert plain_model.greedy_token([0.5, 2.0, 2.0, -1.0]) == 1
    assert plain_model.greedy_token([0.5, float("nan")]) == -1
    assert plain_model.greedy_token([float("-inf")] * 3) == -1
    draws = [plain_model.uniform_number(3, key, step) for key in range(40) for step in range(25)]
    assert all(0.0 <= u < 1.0 for u in draws) and 0.45 < sum(draws) / len(draws) < 0.55
    assert len(set(draws)) > 990
    logits = [0.0, 5.0, 0.0]
    picks = [plain_model.temperature_token(logits, 1.0, 1, key, 0) for key in range(300)]
    assert 0.95 < picks.count(1) / 300 <= 1.0
    assert plain_model.temperature_token(logits, 0.0, 1, 0, 0) == 1
