"""The tiny configurations the tests run: they differ in every size and option."""

# Two layers, heads 4 over 2 key/value heads, head width 16 (heads * width == hidden), tied
# embeddings, theta 1e4, eps 1e-6, every layer with full attention.
TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 128,
    "attention_bias": False, "eos_token_id": 7,
}

# Three layers, heads 8 over 2 (group 4), head width 32 (heads * width = 256 != hidden 96),
# odd intermediate and vocabulary, untied head, theta 1e6, eps 1e-5, the middle layer with a
# window of 24 tokens (a ring of one page).
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 8, "num_key_value_heads": 2,
    "head_dim": 32, "intermediate_size": 200, "vocab_size": 389,
    "rope_parameters": {"rope_theta": 1000000.0, "rope_type": "default"},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 256,
    "layer_types": ["full_attention", "sliding_attention", "full_attention"], "sliding_window": 24,
    "eos_token_id": [3, 11],
}

# Four layers, 6 heads over 3 (group 2), head width 48 (a multiple of 16 that is no power of
# two), one key/value head per two heads, windows of 70 tokens (a ring of two pages that wraps
# within 256 positions) on the even layers.
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu",
    "num_hidden_layers": 4, "hidden_size": 72, "num_attention_heads": 6, "num_key_value_heads": 3,
    "head_dim": 48, "intermediate_size": 136, "vocab_size": 301, "rope_theta": 50000.0,
    "rms_norm_eps": 3e-6, "tie_word_embeddings": False, "max_position_embeddings": 320,
    "layer_types": ["sliding_attention", "full_attention", "sliding_attention", "full_attention"],
    "sliding_window": 70,
}

# Five layers, 3 heads over one key/value head (group 3), head width 64: the width at which
# the bfloat16 engine runs prompts through its tensor-memory attention kernel, whose tiles
# are 128 rows; two layers have a window of 150 tokens, whose edge falls inside a tile.
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu",
    "num_hidden_layers": 5, "hidden_size": 80, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 64, "intermediate_size": 152, "vocab_size": 211, "rope_theta": 200000.0,
    "rms_norm_eps": 2e-6, "tie_word_embeddings": True, "max_position_embeddings": 448,
    "layer_types": ["sliding_attention", "full_attention", "full_attention", "sliding_attention", "full_attention"],
    "sliding_window": 150,
}

# One layer, 2 heads over one key/value head, head width 128 (the benchmark model's width:
# its attention kernels, whole-model), full attention, untied head.
TINY_E = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu",
    "num_hidden_layers": 1, "hidden_size": 160, "num_attention_heads": 2, "num_key_value_heads": 1,
    "head_dim": 128, "intermediate_size": 168, "vocab_size": 307, "rope_theta": 300000.0,
    "rms_norm_eps": 5e-6, "tie_word_embeddings": False, "max_position_embeddings": 384,
}

ALL = {"tiny_a": TINY_A, "tiny_b": TINY_B, "tiny_c": TINY_C, "tiny_d": TINY_D, "tiny_e": TINY_E}


LOGIT_SCALE = 8.0


def sharpen_logits(folder: str, factor: float = LOGIT_SCALE) -> None:
    """Multiplies the final norm's weight of a written model folder by `factor`. With weights
    N(0, 0.02) and widths of a hundred the logits of a tiny model stay below one, and an
    error measured against max(1, largest logit) is then an absolute one that hides relative
    faults; scaled, the largest logits are 5 to 10 and errors are relative to them."""
    import os
    from kidi_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    path = os.path.join(folder, "model.safetensors")
    file = SafetensorsFile(path)
    tensors = {name: file.tensor(name).clone() for name in file.names()}
    file.close()
    tensors["model.norm.weight"] = (tensors["model.norm.weight"].float() * factor).to(tensors["model.norm.weight"].dtype)
    os.remove(path)
    write_safetensors(path, tensors, metadata={"format": "pt"})
