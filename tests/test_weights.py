"""safetensors reading and writing, binding by name, one error for everything that does
not fit, random weights (no GPU)."""
import json
import os
import struct

import pytest
import torch

import plain_model
from kidi_b200 import ErrorCode, KidiError, write_random_model
from kidi_b200.engine.model import declared_parameters
from kidi_b200.registry import spec_from_config
from kidi_b200.weights.loader import Checkpoint, TensorDict, bind_parameters
from kidi_b200.weights.random_init import checkpoint_tensors, random_parameters
from kidi_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
from tiny_configs import TINY_A, TINY_B

CPU = torch.device("cpu")


def params_of(config):
    return declared_parameters(spec_from_config(config)[2])


def tensors_of(config, seed=0, dtype=torch.bfloat16):
    return dict(checkpoint_tensors(params_of(config), seed, dtype))


def bind(config, tensors, dtype=torch.bfloat16):
    return bind_parameters(params_of(config), TensorDict(tensors), engine_dtype=dtype, device=CPU)


def test_round_trip_through_a_file(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
               "c": torch.arange(6, dtype=torch.int32).reshape(2, 3), "empty": torch.zeros(0, 4)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, tensors, metadata={"format": "pt"})
    file = SafetensorsFile(path)
    assert set(file.names()) == set(tensors)
    for name, tensor in tensors.items():
        assert file.dtype(name) == tensor.dtype and file.shape(name) == tuple(tensor.shape)
        assert torch.equal(file.tensor(name), tensor)
    # The independent reader of the safetensors package sees the same file.
    from safetensors.torch import load_file
    other = load_file(path)
    assert all(torch.equal(other[name], tensor) for name, tensor in tensors.items())
    with pytest.raises(KidiError) as caught:  # exclusive create
        write_safetensors(path, tensors)
    assert caught.value.code == ErrorCode.IO


def _file_with_header(tmp_path, header: dict, payload: bytes = b"", name="bad.safetensors", raw_header=None):
    encoded = raw_header if raw_header is not None else json.dumps(header).encode()
    path = tmp_path / name
    path.write_bytes(struct.pack("<Q", len(encoded)) + encoded + payload)
    return str(path)


def test_malformed_files_are_rejected(tmp_path):
    cases = {
        "short": lambda: (tmp_path / "short.safetensors").write_bytes(b"abc") and str(tmp_path / "short.safetensors"),
        "header longer than the file": lambda: _file_with_header(tmp_path, {}, raw_header=b"{}")[:0] or str(
            (tmp_path / "long.safetensors").write_bytes(struct.pack("<Q", 1000) + b"{}") and tmp_path / "long.safetensors"),
        "not json": lambda: _file_with_header(tmp_path, {}, raw_header=b"{nope"),
        "unknown dtype": lambda: _file_with_header(
            tmp_path, {"t": {"dtype": "F7", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 4),
        "span mismatch": lambda: _file_with_header(
            tmp_path, {"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 8),
        "beyond payload": lambda: _file_with_header(
            tmp_path, {"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 8),
        "negative dimension": lambda: _file_with_header(
            tmp_path, {"t": {"dtype": "F32", "shape": [-1], "data_offsets": [0, 0]}}),
        "duplicate name": lambda: _file_with_header(
            tmp_path, {}, b"\0" * 8, raw_header=b'{"t":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},'
                                                b'"t":{"dtype":"F32","shape":[1],"data_offsets":[4,8]}}'),
        "missing field": lambda: _file_with_header(tmp_path, {"t": {"dtype": "F32", "shape": [1]}}),
        "overlapping tensors": lambda: _file_with_header(
            tmp_path, {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                       "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12, name="overlap.safetensors"),
    }
    for what, make in cases.items():
        path = make()
        with pytest.raises(KidiError) as caught:
            SafetensorsFile(path)
        assert caught.value.code == ErrorCode.INVALID_MANIFEST, what


def test_names_follow_the_checkpoint_convention():
    names = set(tensors_of(TINY_B))
    assert "model.embed_tokens.weight" in names and "model.norm.weight" in names and "lm_head.weight" in names
    for layer in range(3):
        for part in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                     "self_attn.q_norm", "self_attn.k_norm", "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj",
                     "input_layernorm", "post_attention_layernorm"):
            assert f"model.layers.{layer}.{part}.weight" in names
    assert "lm_head.weight" not in tensors_of(TINY_A)  # tied: the file does not carry the head


def test_fused_parameters_are_assembled_and_pre_fused_files_pass():
    tensors = tensors_of(TINY_B)
    bound = bind(TINY_B, tensors)
    q, k, v = (tensors[f"model.layers.1.self_attn.{p}_proj.weight"] for p in "qkv")
    fused = bound["model.layers.1.self_attn.qkv_proj.weight"]
    assert fused.shape == (8 * 32 + 2 * 2 * 32, 96)
    assert torch.equal(fused, torch.cat([q, k, v], dim=0))
    gate_up = bound["model.layers.2.mlp.gate_up_proj.weight"]
    assert torch.equal(gate_up, torch.cat([tensors["model.layers.2.mlp.gate_proj.weight"],
                                           tensors["model.layers.2.mlp.up_proj.weight"]], dim=0))
    pre_fused = {name: t for name, t in tensors.items() if "layers.1.self_attn" not in name or "norm" in name
                 or "o_proj" in name}
    pre_fused["model.layers.1.self_attn.qkv_proj.weight"] = fused
    again = bind(TINY_B, pre_fused)
    assert torch.equal(again["model.layers.1.self_attn.qkv_proj.weight"], fused)


def test_dtype_policy():
    tensors = tensors_of(TINY_A)
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()   # stored in 32-bit: stays so
    bound = bind(TINY_A, tensors, torch.bfloat16)
    assert bound["model.norm.weight"].dtype == torch.float32
    assert bound["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16
    widened = bind(TINY_A, tensors, torch.float32)
    assert all(t.dtype == torch.float32 for t in widened.values())
    assert torch.equal(widened["model.layers.0.mlp.down_proj.weight"],
                       tensors["model.layers.0.mlp.down_proj.weight"].float())


def test_wider_checkpoints_in_a_bfloat16_engine():
    """float16 and float32 files: every tensor keeps a width that holds it exactly (32-bit) and
    a warning names the consequence; on request the matrices are rounded to bfloat16 and the
    norm vectors stay 32-bit."""
    for stored in (torch.float16, torch.float32):
        tensors = {name: tensor.to(stored) for name, tensor in tensors_of(TINY_A).items()}
        with pytest.warns(UserWarning, match="32-bit kernel"):
            kept = bind(TINY_A, tensors, torch.bfloat16)
        assert all(tensor.dtype == torch.float32 for tensor in kept.values())
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("error")
            cast = bind_parameters(params_of(TINY_A), TensorDict(tensors), engine_dtype=torch.bfloat16, device=CPU,
                                   cast_matrices=True)
        for name, tensor in cast.items():
            assert tensor.dtype == (torch.bfloat16 if tensor.dim() >= 2 else torch.float32), name
        assert torch.equal(cast["model.layers.0.self_attn.o_proj.weight"],
                           tensors["model.layers.0.self_attn.o_proj.weight"].to(torch.bfloat16))


def test_weight_rules_rename_split_transpose_identical_and_ignore():
    """Each declarative rule of `WeightRule` fills a parameter from a checkpoint that stores it
    under another name or in another layout (src/kidi/checkpoint/weights.h:20-31)."""
    from kidi_b200.parts.spec import ParamSpec, concatenated, identical, renamed, split_from, transposed
    fused = torch.arange(7 * 4, dtype=torch.float32).reshape(7, 4)
    stored = {
        "p.old_name": torch.ones(3, 2),
        "p.fused": fused,
        "p.stored_transposed": torch.arange(6, dtype=torch.float32).reshape(2, 3),
        "p.left": torch.zeros(2, 2), "p.right": torch.ones(2, 3),
        "p.scale_a": torch.full((1,), 0.5), "p.scale_b": torch.full((1,), 0.5),
    }
    params = [
        ("p.", ParamSpec("new_name", (3, 2), rules=(renamed("old_name", (3, 2)),))),
        ("p.", ParamSpec("first", (3, 4), rules=(split_from("fused", (7, 4), 0, 0, 3),))),
        ("p.", ParamSpec("second", (4, 4), rules=(split_from("fused", (7, 4), 0, 3, 4),))),
        ("p.", ParamSpec("columns", (7, 2), rules=(split_from("fused", (7, 4), 1, 2, 2),))),
        ("p.", ParamSpec("matrix", (3, 2), rules=(transposed("stored_transposed", (2, 3)),))),
        ("p.", ParamSpec("wide", (2, 5), rules=(concatenated((("left", (2, 2)), ("right", (2, 3))), axis=1),))),
        ("p.", ParamSpec("scale", (1,), rules=(identical((("scale_a", (1,)), ("scale_b", (1,)))),))),
    ]
    bound = bind_parameters(params, TensorDict(stored), engine_dtype=torch.float32, device=CPU)
    assert torch.equal(bound["p.new_name"], stored["p.old_name"])
    assert torch.equal(bound["p.first"], fused[:3]) and torch.equal(bound["p.second"], fused[3:])
    assert torch.equal(bound["p.columns"], fused[:, 2:4]) and bound["p.columns"].is_contiguous()
    assert torch.equal(bound["p.matrix"], stored["p.stored_transposed"].t())
    assert torch.equal(bound["p.wide"], torch.cat([stored["p.left"], stored["p.right"]], dim=1))
    assert float(bound["p.scale"]) == 0.5
    # Sources that must be identical and are not: refused.
    with pytest.raises(KidiError) as caught:
        bind_parameters(params, TensorDict(dict(stored, **{"p.scale_b": torch.full((1,), 0.25)})),
                        engine_dtype=torch.float32, device=CPU)
    assert "same values" in caught.value.message
    # A tensor nobody uses is unexpected unless a pattern says it may be ignored.
    extra = dict(stored, **{"p.rotary.inv_freq": torch.zeros(4)})
    with pytest.raises(KidiError) as caught:
        bind_parameters(params, TensorDict(extra), engine_dtype=torch.float32, device=CPU)
    assert "unexpected" in caught.value.message and "p.rotary.inv_freq" in caught.value.message
    bind_parameters(params, TensorDict(extra), engine_dtype=torch.float32, device=CPU, ignored=[r"^p\.rotary\."])
    # An absent source of a rule is reported under its own name; a rule that does not make the
    # parameter's shape is a fault of the part that declared it.
    lacking = {name: tensor for name, tensor in stored.items() if name != "p.right"}
    with pytest.raises(KidiError) as caught:
        bind_parameters(params, TensorDict(lacking), engine_dtype=torch.float32, device=CPU)
    assert "missing tensors (1): p.right" in caught.value.message
    with pytest.raises(KidiError) as caught:
        bind_parameters([("p.", ParamSpec("bad", (5, 5), rules=(transposed("stored_transposed", (2, 3)),)))],
                        TensorDict(stored), engine_dtype=torch.float32, device=CPU)
    assert caught.value.code == ErrorCode.INVALID_ARGUMENT


def test_parts_name_tensors_they_ignore():
    """A part's own `ignored_tensors` (relative to its prefix) reach the loader through the model."""
    from kidi_b200.engine.model import CausalLM
    model = CausalLM(spec_from_config(TINY_A)[2], torch.bfloat16, CPU)
    assert model.ignored_tensors() == []
    mixer = model.layers[1].mixer
    mixer.ignored_tensors = lambda: (r"rotary_emb\.inv_freq$",)
    patterns = model.ignored_tensors()
    assert patterns == [r"^model\.layers\.1\.self_attn\.rotary_emb\.inv_freq$"]
    tensors = dict(tensors_of(TINY_A), **{"model.layers.1.self_attn.rotary_emb.inv_freq": torch.zeros(8)})
    bind_parameters(model.parameters(), TensorDict(tensors), engine_dtype=torch.bfloat16, device=CPU, ignored=patterns)
    with pytest.raises(KidiError):
        bind_parameters(model.parameters(), TensorDict(tensors), engine_dtype=torch.bfloat16, device=CPU)


def test_sharded_folder(tmp_path):
    """A folder whose tensors are spread over shards named by model.safetensors.index.json binds
    like the single file; a tensor in two shards and a shard path that leaves the folder are
    refused."""
    tensors = tensors_of(TINY_B)
    names = sorted(tensors)
    cut = len(names) // 3
    shards = {"model-00001-of-00003.safetensors": names[:cut], "model-00002-of-00003.safetensors": names[cut:2 * cut],
              "model-00003-of-00003.safetensors": names[2 * cut:]}
    folder = tmp_path / "sharded"
    folder.mkdir()
    weight_map = {}
    for file, members in shards.items():
        write_safetensors(str(folder / file), {name: tensors[name] for name in members})
        weight_map.update({name: file for name in members})
    (folder / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    checkpoint = Checkpoint(str(folder))
    assert set(checkpoint.names()) == set(names) and len(checkpoint.files) == 3
    bound = bind_parameters(params_of(TINY_B), checkpoint, engine_dtype=torch.bfloat16, device=CPU)
    whole = bind(TINY_B, tensors)
    assert set(bound) == set(whole) and all(torch.equal(bound[name], whole[name]) for name in whole)
    checkpoint.close()
    # The same tensor in two shards.
    write_safetensors(str(folder / "model-00004-of-00003.safetensors"), {names[0]: tensors[names[0]]})
    (folder / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": dict(weight_map, extra="model-00004-of-00003.safetensors")}))
    with pytest.raises(KidiError) as caught:
        Checkpoint(str(folder))
    assert "two shards" in caught.value.message
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "../outside.safetensors"}}))
    with pytest.raises(KidiError) as caught:
        Checkpoint(str(folder))
    assert caught.value.code == ErrorCode.INVALID_MANIFEST


def test_tied_head_shares_storage_and_conflicts_are_rejected():
    tensors = tensors_of(TINY_A)
    bound = bind(TINY_A, tensors)
    assert bound["lm_head.weight"].data_ptr() == bound["model.embed_tokens.weight"].data_ptr()
    same = dict(tensors, **{"lm_head.weight": tensors["model.embed_tokens.weight"].clone()})
    assert bind(TINY_A, same)["lm_head.weight"].data_ptr() == bind(TINY_A, same)["lm_head.weight"].data_ptr()
    other = dict(tensors, **{"lm_head.weight": tensors["model.embed_tokens.weight"] + 1})
    with pytest.raises(KidiError) as caught:
        bind(TINY_A, other)
    assert "tied" in caught.value.message


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    tensors = tensors_of(TINY_B)
    del tensors["model.layers.0.self_attn.k_proj.weight"]
    del tensors["lm_head.weight"]
    tensors["model.layers.9.mlp.up_proj.weight"] = torch.zeros(2, 2, dtype=torch.bfloat16)
    tensors["rotary.inv_freq"] = torch.zeros(4)
    tensors["model.norm.weight"] = torch.zeros(95, dtype=torch.bfloat16)
    tensors["model.layers.2.mlp.down_proj.weight"] = torch.zeros(96, 201, dtype=torch.bfloat16)
    tensors["model.layers.1.input_layernorm.weight"] = torch.zeros(96, dtype=torch.int32)
    with pytest.raises(KidiError) as caught:
        bind(TINY_B, tensors)
    message = caught.value.message
    assert caught.value.code == ErrorCode.INVALID_MANIFEST
    assert "missing tensors (2)" in message and "model.layers.0.self_attn.k_proj.weight" in message
    assert "lm_head.weight" in message
    assert "unexpected tensors (2)" in message and "model.layers.9.mlp.up_proj.weight" in message
    assert "rotary.inv_freq" in message
    assert "wrong shapes or types (3)" in message
    assert "model.norm.weight: shape [95] in the file, [96] expected" in message
    assert "model.layers.2.mlp.down_proj.weight: shape [96, 201]" in message
    assert "model.layers.1.input_layernorm.weight: dtype torch.int32" in message


def test_random_model_folder(tmp_path):
    folder = write_random_model(TINY_B, str(tmp_path / "m"), seed=3)
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    config, tensors = plain_model.read_model_folder(folder)
    assert config["vocab_size"] == 389 and config["torch_dtype"] == "bfloat16"
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())
    # The distributions: matrices ~ N(0, 0.02), norm weights ~ 1 + N(0, 0.1).
    matrix = tensors["model.layers.0.mlp.up_proj.weight"].float()
    assert abs(float(matrix.mean())) < 2e-3 and abs(float(matrix.std()) - 0.02) < 2e-3
    norm = tensors["model.layers.0.input_layernorm.weight"].float()
    assert abs(float(norm.mean()) - 1.0) < 0.05 and 0.05 < float(norm.std()) < 0.15
    # The same seed gives the same folder, another seed another one; a tensor does not
    # depend on which others exist.
    again = plain_model.read_model_folder(write_random_model(TINY_B, str(tmp_path / "n"), seed=3))[1]
    other = plain_model.read_model_folder(write_random_model(TINY_B, str(tmp_path / "o"), seed=4))[1]
    assert all(torch.equal(again[name], tensor) for name, tensor in tensors.items())
    assert not torch.equal(other["model.norm.weight"], tensors["model.norm.weight"])
    # The checkpoint binds, and filling a model in place gives the same values.
    checkpoint = Checkpoint(folder)
    bound = bind_parameters(params_of(TINY_B), checkpoint, engine_dtype=torch.bfloat16, device=CPU)
    direct = random_parameters(params_of(TINY_B), 3, torch.bfloat16, CPU)
    assert set(bound) == set(direct)
    assert all(torch.equal(bound[name], direct[name]) for name in bound)


def test_missing_weights_file(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    with pytest.raises(KidiError) as caught:
        Checkpoint(str(tmp_path))
    assert caught.value.code == ErrorCode.IO
