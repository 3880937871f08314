"""bench.py's record, on a one-layer stack of the benchmark's layer sizes: the keys a reader of the
line relies on, a flat configuration, the checks that vouch for the timed steps, and the two
calls that must not run a benchmark (more than one GPU, the reference arm)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*arguments):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *arguments], capture_output=True, text=True,
                          timeout=600)


@pytest.mark.gpu
def test_the_record_of_a_short_run():
    done = run_bench("--layers", "1", "--steps", "4", "--warmup", "3")
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [line for line in done.stdout.splitlines() if line.strip()]
    assert len(lines) == 1                                    # one JSON line and nothing else on standard output
    record = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches", "roofline", "prefill",
                "points", "checked", "check", "impl"):
        assert key in record, key
    assert record["n_gpus"] == 1 and record["steps"] == 4 and record["warmup"] == 3 and record["dtype"] == "bf16"
    assert record["higher_is_better"] is True and record["impl"] == "ours" and record["checked"] is True
    config = record["config"]
    assert len(config) <= 20 and all(not isinstance(value, (dict, list)) for value in config.values())
    assert config["layers"] == 1 and config["layers_of_model"] == 36       # fewer layers are named beside the model's
    assert config["hidden_size"] == 4096 and config["intermediate_size"] == 12288 and config["global_batch"] == 8
    assert record["check"]["repeats"] >= 3 and record["check"]["repeats_identical"] is True
    assert record["value"] > 0 and abs(record["value"] * record["ms_per_step"] / 1e3 / 8 - 1.0) < 1e-3   # tokens/s = batch / step time
    assert record["gpu_launches"] > 0
    assert set(record["e2e"]) >= {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"}
    assert record["e2e"]["d2h_bytes_per_step"] == 32 and record["e2e"]["value"] > 0
    roofline = record["roofline"]
    assert roofline["bound"] == "hbm" and roofline["unit"] == "GB/s"
    assert abs(roofline["frac"] - roofline["achieved"] / roofline["peak"]) < 1e-3 and 0 < roofline["frac"] < 1.1
    assert set(record["prefill"]) >= {"value", "tokens", "ms", "frac"} and record["prefill"]["tokens"] == 2048
    assert set(record["points"]) == {"decode_b1", "decode_b64"}
    assert set(record["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons"}


def test_more_than_one_gpu_is_refused_and_the_reference_arm_says_why_it_is_not_there():
    several = run_bench("--gpus", "2")
    assert several.returncode == 2 and len(several.stdout.strip().splitlines()) == 1
    reference = run_bench("--impl", "reference")
    assert reference.returncode == 0
    record = json.loads(reference.stdout.strip())
    assert record["impl"] == "reference" and record["unavailable"]
