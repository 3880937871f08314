"""The command line's exit codes and the Python entry point (no GPU), after the
reference's tests/python_cli_test.py:59-118: help 0, bad option 2, missing model 1."""
import json
import subprocess
import sys
import os

import kidi_b200
from tiny_configs import TINY_A

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_entry_point_exit_codes(tmp_path, capsys):
    assert kidi_b200.main(["--help"]) == 0
    assert kidi_b200.main(["generate", "--help"]) == 0
    assert kidi_b200.main([]) == 2
    assert kidi_b200.main(["generate"]) == 2                                  # -m is required
    assert kidi_b200.main(["generate", "-m", "x", "--no-such-option"]) == 2
    assert kidi_b200.main(["generate", "-m", "x", "--precision", "int3"]) == 2
    assert kidi_b200.main(["inspect", "-m", str(tmp_path / "nowhere")]) == 1      # missing model
    assert kidi_b200.main(["generate", "-m", str(tmp_path / "nowhere")]) == 1
    capsys.readouterr()


def test_random_model_and_inspect(tmp_path, capsys):
    config = tmp_path / "config.json"
    config.write_text(json.dumps(TINY_A))
    out = tmp_path / "model"
    assert kidi_b200.main(["random-model", "--config", str(config), "--seed", "2", "-o", str(out)]) == 0
    assert sorted(os.listdir(out)) == ["config.json", "model.safetensors"]
    capsys.readouterr()
    assert kidi_b200.main(["inspect", "-m", str(out)]) == 0
    text = capsys.readouterr().out
    assert "architecture: Qwen3ForCausalLM" in text and "layers: 2" in text
    # Without a GPU generation fails loudly with a runtime fault, not with a wrong answer.
    import torch
    if not torch.cuda.is_available():
        requests = tmp_path / "in.jsonl"
        requests.write_text(json.dumps({"token_ids": [1, 2, 3]}) + "\n")
        assert kidi_b200.main(["generate", "-m", str(out), "-i", str(requests)]) == 1
        assert "CUDA" in capsys.readouterr().err


def test_module_and_script_run(tmp_path):
    for command in ([sys.executable, "-m", "kidi_b200", "--help"], [sys.executable, os.path.join(ROOT, "bin", "kidi_b200"), "--help"]):
        result = subprocess.run(command, capture_output=True, text=True, cwd=ROOT)
        assert result.returncode == 0 and "generate" in result.stdout
    result = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run")], capture_output=True, text=True)
    assert result.returncode == 2 and "--model" in result.stderr
