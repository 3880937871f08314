"""Random configurations of middle size with prompts of one to three thousand tokens, against the
plain model: the kernels that only many rows reach in a whole model (the tcgen05 matrix product
from 1,024 rows on, tcgen05 prompt attention at head widths 64 and 128 and the mma.sync kernel
at others, prompts that continue a cached sequence, windows of hundreds of tokens), at widths
and lengths that are no round numbers, in 32-bit and in bfloat16."""
import numpy as np
import pytest
import torch

import replay_helpers as rh

pytestmark = pytest.mark.gpu


def random_config(rng):
    kv_heads = int(rng.choice([1, 2, 4]))
    layers = int(rng.integers(1, 3))
    types = ["full_attention"] * layers
    window = None
    if rng.random() < 0.4:
        window = int(rng.integers(70, 1500))
        types = ["sliding_attention" if rng.random() < 0.6 else "full_attention" for _ in range(layers)]
    config = {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu",
        "num_hidden_layers": layers, "hidden_size": int(rng.choice([256, 320, 512, 520, 768, 1000, 1024])),
        "num_attention_heads": kv_heads * int(rng.choice([1, 2, 4, 6, 8])), "num_key_value_heads": kv_heads,
        "head_dim": int(rng.choice([64, 128, 128, 32, 96])),
        "intermediate_size": int(rng.choice([256, 520, 1024, 1536, 2000])),
        "vocab_size": int(rng.integers(500, 3000)), "rope_theta": float(rng.choice([1e4, 1e6])),
        "rms_norm_eps": 1e-6, "tie_word_embeddings": bool(rng.random() < 0.5),
        "max_position_embeddings": 3072, "layer_types": types,
    }
    if "sliding_attention" in types:
        config["sliding_window"] = window
    return config


@pytest.mark.parametrize("seed", [1, 5, 6, 7])     # a window at width 64; width 96; 16 heads over 4; hidden 520
def test_a_random_configuration_of_middle_size(tmp_path, record_property, seed):
    from tiny_configs import sharpen_logits
    from kidi_b200 import Engine, write_random_model
    from kidi_b200.kernels import ops
    rng = np.random.default_rng(5000 + seed)
    config = random_config(rng)
    lengths = sorted({int(rng.integers(1, 60)), int(rng.integers(900, 1100)), int(rng.integers(1024, 2200)),
                      int(rng.integers(2200, 3072))})
    folder = write_random_model(config, str(tmp_path / "model"), seed=seed, dtype=torch.bfloat16)
    sharpen_logits(folder)
    requests = rh.random_requests(config["vocab_size"], lengths, seed=seed)
    expected = rh.plain_logits(folder, requests)
    # Within three times the largest differences measured on a B200: 2.1e-6 and 8.7e-3 on these four
    # configurations' whole prompts, 3.1e-6 and 1.24e-2 over 130 configurations drawn this way, every cut.
    for dtype, tolerance in (("float32", 7e-6), ("bfloat16", 2.9e-2)):
        what = f"seed {seed}, {dtype}"
        engine = Engine.load(folder, dtype=dtype, max_tokens=16384)
        with ops.record_launches() as names:
            whole = rh.run_whole(engine, requests)
        record_property(f"max_error_{dtype}", rh.worst_error(whole, expected))
        rh.assert_matches(whole, expected, tolerance, what + ": whole")
        rh.assert_matches(rh.run_tail_decoded(engine, requests, 8), expected, tolerance, what + ": last 8 one by one")
        rh.assert_matches(rh.run_chunked(engine, requests, chunk=1100), expected, tolerance, what + ": chunks of 1,100")
        if dtype == "bfloat16":
            assert "gemm_tcgen05" in names, sorted(set(names))       # the longest prompt has over 1,024 rows
            assert any(name.startswith("attention_prefill") for name in names), sorted(set(names))
        engine.cache.check()
        assert not engine.cache.slots.held
        engine.check_device_errors()
        del engine
        torch.cuda.empty_cache()
