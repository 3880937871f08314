"""Dense Qwen3 as a `ModelSpec`.

Layer math and tensor names are the reference's: a pre-norm block with two residual
adds (src/kidi/layers/qwen3.cpp:100-122), grouped-query attention whose q and k
heads pass a per-head RMSNorm and then rotary position encoding
(src/kidi/layers/qwen3.cpp:13-56), a SiLU-gated feed-forward
(src/kidi/layers/gemma4.cpp:164-225), token embedding with scale 1 and a final
RMSNorm (src/kidi/model/qwen3.cpp:69-99), loaded from the Hugging Face names the
reference's round-trip test proves (tests/kidi/model/qwen3_test.cpp:111-141). The
causal mask, the cache, the output head and `tie_word_embeddings` are this
library's own: the reference's Qwen3 is a bidirectional backbone
(src/kidi/model/qwen3.cpp:165-167) without them.

This file is the whole of what is architecture-specific: it maps a `Qwen3Config` to
parts and their parameters. Another architecture is another file like it.
"""
from __future__ import annotations

from ..config.qwen3 import SLIDING_ATTENTION, Qwen3Config
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..registry import register_architecture


def build_spec(config: Qwen3Config) -> ModelSpec:
    hidden = config.hidden_size
    norm = {"size": hidden, "eps": config.rms_norm_eps}
    layers = []
    for index, layer_type in enumerate(config.layer_types):
        prefix = f"model.layers.{index}."
        window = config.sliding_window if layer_type == SLIDING_ATTENTION else None
        layers.append(LayerSpec(
            arrangement=PartSpec("pre_norm"),
            parts={
                "input_norm": PartSpec("rms_norm", norm, prefix + "input_layernorm."),
                "mixer": PartSpec("attention", {
                    "hidden_size": hidden,
                    "num_heads": config.num_attention_heads,
                    "num_kv_heads": config.num_key_value_heads,
                    "head_dim": config.head_dim,
                    "qk_norm": True,
                    "qk_norm_eps": config.rms_norm_eps,
                    "position": "rope",
                    "window": window,
                }, prefix + "self_attn."),
                "post_norm": PartSpec("rms_norm", norm, prefix + "post_attention_layernorm."),
                "feed_forward": PartSpec("gated_mlp", {
                    "hidden_size": hidden,
                    "intermediate_size": config.intermediate_size,
                    "activation": "silu",
                }, prefix + "mlp."),
            },
        ))
    return ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab_size,
        hidden_size=hidden,
        max_positions=config.max_position_embeddings,
        embedding=PartSpec("token_embedding", {
            "vocab_size": config.vocab_size, "hidden_size": hidden, "scale": 1.0,
        }, "model.embed_tokens."),
        positions={"rope": PartSpec("rotary", {
            "head_dim": config.head_dim,
            "rotary_dim": config.head_dim,
            "theta": config.rope_theta,
            "max_positions": config.max_position_embeddings,
        })},
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(index) for index in range(len(layers))),
        final_norm=PartSpec("rms_norm", norm, "model.norm."),
        head=PartSpec("linear_head", {
            "hidden_size": hidden,
            "vocab_size": config.vocab_size,
            "tied_to": "model.embed_tokens.weight" if config.tie_word_embeddings else None,
        }, "lm_head."),
        eos_token_ids=config.eos_token_ids,
    )


register_architecture("Qwen3ForCausalLM", Qwen3Config, build_spec, aliases=("qwen3",))
