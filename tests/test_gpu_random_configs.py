"""Random tiny configurations through the engine against the plain model: sizes that no
hand-picked configuration has (odd widths and vocabularies, head widths that are no
multiple of 16, up to 17 query heads per key/value head, windows of any length), in
32-bit and in bfloat16, every way of cutting. A size is either computed right or refused
with an error of the package's own; it never gives a wrong result."""
import numpy as np
import pytest
import torch

import replay_helpers as rh

pytestmark = pytest.mark.gpu

HEAD_DIMS = (16, 32, 48, 64, 128, 192, 256)      # the tensor-core attention kernels
OTHER_HEAD_DIMS = (2, 6, 10, 24, 40, 72, 100)    # even, no multiple of 16: the general kernels


def random_config(rng):
    head_dim = int(rng.choice(OTHER_HEAD_DIMS if rng.random() < 0.25 else HEAD_DIMS))
    kv_heads = int(rng.choice([1, 1, 2, 3, 4, 5]))
    group = int(rng.choice([1, 2, 3, 4, 5, 6, 7, 8, 9, 12, 16, 17]))
    while kv_heads * group * head_dim > 4096:
        group = max(1, group // 2)
    layers = int(rng.integers(1, 4))
    max_positions = int(rng.choice([96, 200, 330, 520]))
    types = ["full_attention"] * layers
    window = None
    if rng.random() < 0.5:
        window = int(rng.integers(3, 180))
        types = ["sliding_attention" if rng.random() < 0.6 else "full_attention" for _ in range(layers)]
    config = {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu",
        "num_hidden_layers": layers, "hidden_size": int(rng.choice([24, 37, 40, 50, 64, 66, 72, 90, 100, 136, 200, 255])),
        "num_attention_heads": kv_heads * group, "num_key_value_heads": kv_heads, "head_dim": head_dim,
        "intermediate_size": int(rng.choice([16, 33, 50, 100, 136, 200, 257, 301])),
        "vocab_size": int(rng.integers(50, 1200)), "rope_theta": float(rng.choice([1e4, 5e4, 1e6])),
        "rms_norm_eps": float(rng.choice([1e-6, 3e-6, 1e-5])), "tie_word_embeddings": bool(rng.random() < 0.5),
        "max_position_embeddings": max_positions, "layer_types": types,
    }
    if "sliding_attention" in types:
        config["sliding_window"] = window
    return config


@pytest.mark.parametrize("seed", range(12))
def test_a_random_configuration(tmp_path, record_property, seed):
    from tiny_configs import sharpen_logits
    from kidi_b200 import Engine, write_random_model
    rng = np.random.default_rng(1000 + seed)
    config = random_config(rng)
    top = config["max_position_embeddings"]
    lengths = sorted({1, int(rng.integers(2, 40)), int(rng.integers(40, top)), int(rng.integers(top // 2, top)), top})
    folder = write_random_model(config, str(tmp_path / "model"), seed=seed, dtype=torch.bfloat16)
    sharpen_logits(folder)        # largest logits of 5 to 10: differences are relative to them
    requests = rh.random_requests(config["vocab_size"], lengths, seed=seed)
    expected = rh.plain_logits(folder, requests)
    sizes = {key: config[key] for key in ("hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                                          "intermediate_size", "vocab_size", "layer_types")}
    # Three times the largest differences measured over these twelve configurations on a B200
    # (1.9e-6 and 7.0e-3; every run records its own: `record_property`).
    for dtype, tolerance in (("float32", 6e-6), ("bfloat16", 2.1e-2)):
        what = f"{sizes}, window {config.get('sliding_window')}, {dtype}"
        engine = Engine.load(folder, dtype=dtype, max_tokens=4096)
        whole = rh.run_whole(engine, requests)
        record_property(f"max_error_{dtype}", rh.worst_error(whole, expected))
        record_property(f"rms_error_{dtype}", rh.rms_error(whole, expected))
        rh.assert_matches(whole, expected, tolerance, what + ": whole")
        rh.assert_matches(rh.run_tail_decoded(engine, requests, 20), expected, tolerance, what + ": last 20 one by one")
        rh.assert_matches(rh.run_batches(engine, requests, batch_size=3), expected, tolerance, what + ": batches of 3")
        rh.assert_matches(rh.run_chunked(engine, requests, chunk=70), expected, tolerance, what + ": chunks of 70")
        engine.cache.check()
        assert not engine.cache.slots.held
        tokens = engine.generate([tokens[:5] for tokens in list(requests.values())[1:4]], max_new_tokens=4, ignore_eos=True)
        assert all(len(found) == 4 for found in tokens)
        engine.check_device_errors()
