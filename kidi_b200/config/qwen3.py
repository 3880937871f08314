"""Typed configuration of dense Qwen3, read from the model's own config.json keys.

Keys and validation follow the reference (src/kidi/model/qwen3.cpp:38-67): every
size is required and positive, heads divide into key/value heads, head_dim is even,
eps and theta are finite and positive, hidden_act is "silu". Beyond the reference
(which has no output head and rejects every layer type but "full_attention",
src/kidi/model/qwen3.cpp:59-62) this reads `tie_word_embeddings`, a flat
`rope_theta` when `rope_parameters` is absent, and `sliding_window` for layers whose
`layer_types` entry is "sliding_attention".
"""
from __future__ import annotations

import dataclasses
from typing import Any, Mapping, Optional, Tuple

from ..errors import invalid_manifest, unsupported
from .reader import ConfigReader

FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"


@dataclasses.dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    layer_types: Tuple[str, ...]
    sliding_window: Optional[int]
    eos_token_ids: Tuple[int, ...]

    architecture = "Qwen3ForCausalLM"
    model_type = "qwen3"

    @classmethod
    def from_dict(cls, values: Mapping[str, Any]) -> "Qwen3Config":
        reader = ConfigReader(values)
        model_type = reader.string("model_type", cls.model_type)
        if model_type != cls.model_type:
            raise invalid_manifest(f"expected model_type 'qwen3', found '{model_type}'")
        if reader.string("hidden_act") != "silu":
            raise invalid_manifest("expected a Qwen3 SiLU configuration (hidden_act must be 'silu')")
        rope = reader.child("rope_parameters")
        if rope is not None:
            theta = rope.number("rope_theta")
            rope_type = rope.string("rope_type", "default")
            if rope_type != "default":
                raise unsupported(f"rope_type '{rope_type}' is not supported (default rotary only)")
        else:
            theta = reader.number("rope_theta")
        scaling = reader.raw("rope_scaling")
        if scaling is not None and not (
            isinstance(scaling, Mapping) and scaling.get("rope_type", scaling.get("type")) == "default"
        ):
            raise unsupported("rope_scaling is not supported (default rotary only)")
        if reader.boolean("attention_bias", False):
            raise unsupported("attention_bias=true is not supported (projections carry no bias)")
        layers = reader.integer("num_hidden_layers")
        layer_types = reader.strings("layer_types", None)
        if layer_types is None:
            layer_types = (FULL_ATTENTION,) * max(layers, 0)
        window = reader.integer("sliding_window", None) if reader.has("sliding_window") else None
        eos = reader.raw("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise invalid_manifest("'eos_token_id' must be an integer or a list of integers")
        config = cls(
            vocab_size=reader.integer("vocab_size"),
            hidden_size=reader.integer("hidden_size"),
            intermediate_size=reader.integer("intermediate_size"),
            num_hidden_layers=layers,
            num_attention_heads=reader.integer("num_attention_heads"),
            num_key_value_heads=reader.integer("num_key_value_heads"),
            head_dim=reader.integer("head_dim"),
            max_position_embeddings=reader.integer("max_position_embeddings"),
            rms_norm_eps=reader.number("rms_norm_eps"),
            rope_theta=theta,
            tie_word_embeddings=reader.boolean("tie_word_embeddings", False),
            layer_types=tuple(layer_types),
            sliding_window=window,
            eos_token_ids=eos_ids,
        )
        config.validate()
        return config

    def validate(self) -> None:
        sizes = (
            self.vocab_size, self.hidden_size, self.intermediate_size, self.num_hidden_layers,
            self.num_attention_heads, self.num_key_value_heads, self.head_dim, self.max_position_embeddings,
        )
        if any(size <= 0 for size in sizes):
            raise invalid_manifest("invalid Qwen3 dimensions: every size must be positive")
        if self.num_attention_heads % self.num_key_value_heads:
            raise invalid_manifest("invalid Qwen3 dimensions: num_attention_heads must be a multiple of num_key_value_heads")
        if self.head_dim % 2:
            raise invalid_manifest("invalid Qwen3 dimensions: head_dim must be even")
        if not self.rms_norm_eps > 0 or not self.rope_theta > 0:
            raise invalid_manifest("invalid Qwen3 dimensions: rms_norm_eps and rope_theta must be positive")
        if len(self.layer_types) != self.num_hidden_layers:
            raise invalid_manifest("layer_types must name every layer")
        for kind in self.layer_types:
            if kind not in (FULL_ATTENTION, SLIDING_ATTENTION):
                raise unsupported(f"layer type '{kind}' is not supported")
        if SLIDING_ATTENTION in self.layer_types and (self.sliding_window is None or self.sliding_window <= 0):
            raise invalid_manifest("sliding_attention layers need a positive 'sliding_window'")
        if any(token < 0 or token >= self.vocab_size for token in self.eos_token_ids):
            raise invalid_manifest("eos_token_id lies outside the vocabulary")

    def to_dict(self) -> dict:
        """The config.json that `from_dict` reads back to an equal configuration."""
        values = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "hidden_act": "silu",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_parameters": {"rope_theta": self.rope_theta, "rope_type": "default"},
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": False,
            "layer_types": list(self.layer_types),
        }
        if self.sliding_window is not None:
            values["sliding_window"] = self.sliding_window
        if self.eos_token_ids:
            values["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return values
