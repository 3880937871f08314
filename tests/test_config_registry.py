"""Configuration and registry (no GPU)."""
import copy
import json

import pytest

from kidi_b200 import ErrorCode, KidiError, register_architecture, registered_architectures
from kidi_b200.config.qwen3 import Qwen3Config
from kidi_b200.config.reader import read_config_json
from kidi_b200.registry import resolve_architecture, spec_from_config
from tiny_configs import ALL, TINY_A, TINY_B


def code_of(callable_, *args):
    with pytest.raises(KidiError) as caught:
        callable_(*args)
    return caught.value.code, caught.value.message


@pytest.mark.parametrize("name", list(ALL))
def test_typed_config_reads_every_key(name):
    raw = ALL[name]
    config = Qwen3Config.from_dict(raw)
    assert config.vocab_size == raw["vocab_size"]
    assert config.hidden_size == raw["hidden_size"]
    assert config.intermediate_size == raw["intermediate_size"]
    assert config.num_hidden_layers == raw["num_hidden_layers"]
    assert config.num_attention_heads == raw["num_attention_heads"]
    assert config.num_key_value_heads == raw["num_key_value_heads"]
    assert config.head_dim == raw["head_dim"]
    assert config.max_position_embeddings == raw["max_position_embeddings"]
    assert config.rms_norm_eps == raw["rms_norm_eps"]
    theta = raw["rope_parameters"]["rope_theta"] if "rope_parameters" in raw else raw["rope_theta"]
    assert config.rope_theta == theta
    assert config.tie_word_embeddings == raw["tie_word_embeddings"]
    assert len(config.layer_types) == raw["num_hidden_layers"]
    # to_dict round-trips to an equal configuration.
    assert Qwen3Config.from_dict(config.to_dict()) == config


def test_the_tiny_configurations_differ_in_every_size():
    keys = ["num_hidden_layers", "hidden_size", "num_attention_heads", "head_dim", "intermediate_size",
            "vocab_size", "rms_norm_eps", "max_position_embeddings"]
    for key in keys:
        assert len({json.dumps(config[key]) for config in ALL.values()}) == len(ALL), key
    groups = {c["num_attention_heads"] // c["num_key_value_heads"] for c in ALL.values()}
    assert len(groups) >= 2
    assert TINY_A["tie_word_embeddings"] != TINY_B["tie_word_embeddings"]


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "num_key_value_heads", "head_dim",
                                 "max_position_embeddings", "rms_norm_eps", "hidden_act"])
def test_a_missing_key_is_an_invalid_manifest(key):
    raw = copy.deepcopy(TINY_A)
    del raw[key]
    code, message = code_of(Qwen3Config.from_dict, raw)
    assert code == ErrorCode.INVALID_MANIFEST and key in message


def test_no_defaults_for_theta():
    raw = copy.deepcopy(TINY_A)
    del raw["rope_theta"]
    assert code_of(Qwen3Config.from_dict, raw)[0] == ErrorCode.INVALID_MANIFEST


@pytest.mark.parametrize("change,code", [
    ({"num_key_value_heads": 3}, ErrorCode.INVALID_MANIFEST),        # 4 heads do not divide into 3
    ({"head_dim": 15}, ErrorCode.INVALID_MANIFEST),                  # odd head width
    ({"vocab_size": 0}, ErrorCode.INVALID_MANIFEST),
    ({"rms_norm_eps": 0.0}, ErrorCode.INVALID_MANIFEST),
    ({"rope_theta": -1.0}, ErrorCode.INVALID_MANIFEST),
    ({"hidden_act": "gelu"}, ErrorCode.INVALID_MANIFEST),
    ({"hidden_size": "64"}, ErrorCode.INVALID_MANIFEST),
    ({"layer_types": ["full_attention"]}, ErrorCode.INVALID_MANIFEST),   # two layers, one entry
    ({"layer_types": ["full_attention", "linear_attention"]}, ErrorCode.UNSUPPORTED),
    ({"layer_types": ["full_attention", "sliding_attention"]}, ErrorCode.INVALID_MANIFEST),  # no window given
    ({"attention_bias": True}, ErrorCode.UNSUPPORTED),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, ErrorCode.UNSUPPORTED),
    ({"eos_token_id": 256}, ErrorCode.INVALID_MANIFEST),
    ({"model_type": "llama"}, ErrorCode.INVALID_MANIFEST),
])
def test_invalid_configurations(change, code):
    raw = copy.deepcopy(TINY_A)
    raw.update(change)
    assert code_of(Qwen3Config.from_dict, raw)[0] == code


def test_registry_chooses_by_architecture_then_model_type():
    assert "Qwen3ForCausalLM" in registered_architectures()
    assert resolve_architecture(TINY_A).name == "Qwen3ForCausalLM"
    only_type = {k: v for k, v in TINY_A.items() if k != "architectures"}
    assert resolve_architecture(only_type).name == "Qwen3ForCausalLM"
    unknown = dict(TINY_A, architectures=["MambaForCausalLM"], model_type="mamba")
    assert code_of(resolve_architecture, unknown)[0] == ErrorCode.UNSUPPORTED
    # A model_type alone that nobody registered is an unsupported model, not a broken manifest
    # (src/kidi/checkpoint/config.cpp:260-264).
    assert code_of(resolve_architecture, {"model_type": "mamba"})[0] == ErrorCode.UNSUPPORTED
    assert code_of(resolve_architecture, {"model_type": 7})[0] == ErrorCode.INVALID_MANIFEST
    assert code_of(resolve_architecture, {"hidden_size": 3})[0] == ErrorCode.INVALID_MANIFEST


def test_spec_carries_the_configuration_and_nothing_else():
    _, typed, spec = spec_from_config(TINY_B)
    assert spec.vocab_size == 389 and spec.hidden_size == 96 and spec.max_positions == 256
    assert len(spec.layers) == 3 and [entry.layer for entry in spec.schedule] == [0, 1, 2]
    windows = [layer.parts["mixer"].param("window") for layer in spec.layers]
    assert windows == [None, 24, None]
    mixer = spec.layers[0].parts["mixer"]
    assert (mixer.param("num_heads"), mixer.param("num_kv_heads"), mixer.param("head_dim")) == (8, 2, 32)
    assert mixer.param("qk_norm_eps") == 1e-5 and spec.final_norm.param("eps") == 1e-5
    assert spec.positions["rope"].param("theta") == 1e6
    assert spec.head.param("tied_to") is None
    assert spec_from_config(TINY_A)[2].head.param("tied_to") == "model.embed_tokens.weight"
    assert spec.eos_token_ids == (3, 11)


def test_a_new_architecture_registers_without_touching_the_package():
    class ToyConfig:
        @classmethod
        def from_dict(cls, values):
            return cls()

    sentinel = object()
    register_architecture("ToyForCausalLM", ToyConfig, lambda config: sentinel, aliases=("toy",))
    assert spec_from_config({"architectures": ["ToyForCausalLM"]})[2] is sentinel
    assert spec_from_config({"model_type": "toy"})[2] is sentinel


def test_config_json_errors(tmp_path):
    assert code_of(read_config_json, str(tmp_path))[0] == ErrorCode.IO
    (tmp_path / "config.json").write_text("{ not json")
    assert code_of(read_config_json, str(tmp_path))[0] == ErrorCode.INVALID_MANIFEST
    (tmp_path / "config.json").write_text("[1, 2]")
    assert code_of(read_config_json, str(tmp_path))[0] == ErrorCode.INVALID_MANIFEST
