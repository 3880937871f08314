"""The arithmetic behind bench.py's record (no GPU): the bytes a decode step has to read and the
floating-point operations of a prefill, against the model's own declared parameters and against
the figures written out by hand for the 8B shape."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench  # noqa: E402


def declared_bytes(config):
    """Bytes of every declared parameter in bfloat16, by name (tied or fused tensors counted once)."""
    from kidi_b200.engine.model import declared_parameters
    from kidi_b200.registry import spec_from_config
    sizes = {}
    for prefix, spec in declared_parameters(spec_from_config(config)[2]):
        if spec.alias_of is None:
            sizes[prefix + spec.name] = 2 * int(np.prod(spec.shape))
    return sizes


def test_decode_bytes_are_the_declared_weights_and_the_live_cache():
    for name in ("8b", "14b", "32b"):
        _, config, batch, _, _ = bench.MODELS[name]
        sizes = declared_bytes(config)
        table = sizes.pop("model.embed_tokens.weight")          # a step reads `batch` rows of it, not the table
        assert table == 2 * config["vocab_size"] * config["hidden_size"]
        weights = sum(sizes.values()) + 2 * batch * config["hidden_size"]
        context = 1039.5
        per_token = 2 * 2 * config["num_hidden_layers"] * config["num_key_value_heads"] * config["head_dim"]
        assert bench.decode_bytes(config, batch, context) == weights + per_token * context * batch, name
    # The 8B shape by hand: 36 layers of 192.9 M weights, a head of 622.3 M; 147,456 cache bytes a token.
    _, config, batch, _, _ = bench.MODELS["8b"]
    found = bench.decode_bytes(config, batch, 1039.5)
    assert abs(found - (15.137e9 + 147456 * 1039.5 * 8)) < 2e6


def test_prefill_operations():
    _, config, _, _, _ = bench.MODELS["8b"]
    tokens = 2048
    sizes = declared_bytes(config)
    matrices = sum(size for name, size in sizes.items() if name.endswith("proj.weight")) // 2   # elements of the layers' products
    linear = 2.0 * tokens * matrices
    attention = config["num_hidden_layers"] * 4.0 * config["num_attention_heads"] * config["head_dim"] * tokens * (tokens + 1) / 2
    head = 2.0 * config["vocab_size"] * config["hidden_size"]                                     # the last row only
    assert bench.prefill_flops(config, tokens) == linear + attention + head
    assert abs(bench.prefill_flops(config, tokens) / 1e12 - 29.69) < 0.05                          # 29.7 TFLOP


def test_peaks_fall_back_when_no_measurement_is_there(tmp_path, monkeypatch):
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    assert bench.peaks()["source"] == "fallback" and bench.peaks()["hbm_gbs"] == 6650.0
    (tmp_path / "MEASURED_PEAKS.json").write_text('{"hbm_gbs": 6000.0, "bf16_tflops": 1500.0}')
    found = bench.peaks()
    assert found == {"hbm_gbs": 6000.0, "bf16_tflops": 1500.0, "bf16_tflops_sustained": 1500.0, "source": "measured"}
