#!/usr/bin/env python3
"""Decode and prefill throughput of the library on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch B] [--model 8b|14b|32b] [--impl ours|reference]

A step is one decode step of the batch. The default run is the Qwen3-8B shape (every
layer size, all 36 layers) with random bfloat16 weights drawn on the device from a
seed, a batch of 8 sequences with 1,024-token prompts of uniform token ids, then 512
decoded tokens each. `--model 14b` and `--model 32b` run the other two shapes with their
batches of unequal prompts (16 prompts of 128 to 2,048 tokens, 8 prompts of 512 to 8,192
tokens; 256 steps). It prints ONE line of JSON:

* `value`: decoded tokens a second, timed on the device with CUDA events over exactly K
  steps after W warm-up steps (tokens selected and fed back on the device): the median
  of three measured repeats of the same prompts, whose token ids must be identical
  (the reference's protocol: benchmarks/README.md:27-35, benchmarks/cuda/run.py:48-49);
* `check`: what vouches for the timed work: the repeats' tokens were identical, and the
  first 16 tokens of the replayed graph are those of plain `Engine.step` calls fed with the
  same inputs (tokens that differ are counted, with the distance of the two candidates'
  logits: the graph may split a sequence's keys otherwise than a single step does, and
  bfloat16 rounding then reorders logits that lie closer together than it);
* `e2e`: the same through the Python entry point (`Engine.generate`): host token ids in
  and out; every step's tokens are read back to pinned host memory for the stop test
  while the next step, fed on the device, already runs;
* `prefill`: one 2,048-token prompt: tokens a second, milliseconds, and the fraction of
  the bfloat16 tensor-core peak its FLOPs reach;
* `roofline`: the decode step's bytes (every weight it uses once, plus the cache of the
  live sequences) over its time, against the measured HBM copy bandwidth;
* `points`: decode tokens a second at batch 1 and 64.

Every decode step reads about 16 GB of weights and cache, far more than the 126 MB L2, so
no L2 flush is needed between timed steps. Peaks come from MEASURED_PEAKS.json beside
this file when the driver wrote it. The reference arm cannot run here: the reference
does not build without its third-party submodules, which are empty in the mounted tree.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu",
    "num_hidden_layers": 36, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 40960, "attention_bias": False,
}
QWEN3_14B = dict(QWEN3_8B, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, intermediate_size=17408)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600)
# name -> (configuration, batch, (shortest, longest) prompt, decode steps): the benchmark's three shapes
MODELS = {
    "8b": ("Qwen3-8B shape", QWEN3_8B, 8, (1024, 1024), 512),
    "14b": ("Qwen3-14B shape", QWEN3_14B, 16, (128, 2048), 256),
    "32b": ("Qwen3-32B shape", QWEN3_32B, 8, (512, 8192), 256),
}
PREFILL_TOKENS = 2048
CHECKED_STEPS = 16
ROUNDING_DISTANCE = 2.5e-2   # of the largest logit: the bfloat16 bound of the benchmark-shape test
REPEATS = 3
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as handle:
            found = json.load(handle)
        hbm = float(found.get("hbm_gbs") or found.get("hbm_gb_s"))
        tflops = float(found.get("bf16_tflops"))
        sustained = float(found.get("bf16_tflops_sustained") or tflops)
        return {"hbm_gbs": hbm, "bf16_tflops": tflops, "bf16_tflops_sustained": sustained, "source": "measured"}
    except (OSError, ValueError, TypeError, KeyError):
        return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.lines, self.process, self.index = [], None, index

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.process = None

    def _read(self):
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.process.terminate()
        clocks, maxima, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            fields = [field.strip() for field in line.split(",")]
            if len(fields) < 6 or not fields[0].isdigit():
                continue
            clocks.append(int(fields[0]))
            maxima.append(int(fields[1]))
            reasons.update(name for name, field in zip(names, fields[2:6]) if field.lower().startswith("active"))
        return {"sm_mhz": statistics.median(clocks) if clocks else None,
                "sm_max_mhz": max(maxima) if maxima else None, "reasons": sorted(reasons), "samples": len(clocks)}


def decode_bytes(config: dict, batch: int, context: float) -> float:
    """Bytes a decode step has to read: every weight it uses once (bfloat16), the
    embedding rows of the batch, and the keys and values of the live sequences."""
    hidden, inter, layers = config["hidden_size"], config["intermediate_size"], config["num_hidden_layers"]
    q = config["num_attention_heads"] * config["head_dim"]
    kv = config["num_key_value_heads"] * config["head_dim"]
    per_layer = hidden * (q + 2 * kv) + q * hidden + 3 * hidden * inter + 2 * hidden + 2 * config["head_dim"]
    weights = 2 * (layers * per_layer + config["vocab_size"] * hidden + hidden + batch * hidden)
    cache = 2 * layers * 2 * kv * context * batch
    return float(weights + cache)


def prefill_flops(config: dict, tokens: int) -> float:
    hidden, inter, layers = config["hidden_size"], config["intermediate_size"], config["num_hidden_layers"]
    q = config["num_attention_heads"] * config["head_dim"]
    kv = config["num_key_value_heads"] * config["head_dim"]
    linear = 2.0 * tokens * layers * (hidden * (q + 2 * kv) + q * hidden + 3 * hidden * inter)
    attention = layers * 4.0 * q * tokens * (tokens + 1) / 2
    head = 2.0 * config["vocab_size"] * hidden
    return linear + attention + head


def draw_prompts(vocab: int, batch: int, lengths, seed: int):
    """`batch` prompts of uniform token ids whose lengths are uniform in [lengths[0], lengths[1]]."""
    import numpy as np
    generator = np.random.default_rng(seed)
    sizes = [lengths[0]] * batch if lengths[0] == lengths[1] else generator.integers(lengths[0], lengths[1] + 1, size=batch)
    return [generator.integers(0, vocab, size=int(size)).tolist() for size in sizes]


def time_decode(engine, sampler, prompts, steps: int, warmup: int, clocks: bool, repeats: int = REPEATS,
                profile_steps: int = 0):
    """Device-timed decode, `repeats` times over: the prompts in one step, then `warmup` +
    `steps` replayed steps with tokens selected and fed back on the device, every step's
    tokens kept on the device. Returns the median repeat's measurements, the tokens of the
    first repeat and whether every repeat produced the same tokens."""
    import torch
    from kidi_b200 import StepBatch
    from kidi_b200.engine.decode_graph import DecodeSession

    batch = len(prompts)
    longest = max(len(prompt) for prompt in prompts) + warmup + steps + 1
    session = DecodeSession(engine, batch, sampler, longest=longest)
    history = torch.zeros((warmup + steps, batch), dtype=torch.int32, device=engine.device)
    runs, tokens_of_repeat, clock_record = [], [], None
    for repeat in range(repeats):
        slots = [engine.acquire() for _ in range(batch)]
        try:
            logits = engine.step(StepBatch(slots, prompts, None))
            first = sampler.select(logits).cpu().tolist()
            session.load(slots, first, [0.0] * batch, list(range(batch)), [1] * batch)
            session.reserve(warmup + steps)
            for step in range(warmup):
                session.launch()
                history[step].copy_(session.selected, non_blocking=True)
            torch.cuda.synchronize()
            sampler_thread = ClockSampler() if clocks and repeat == repeats - 1 else None
            if sampler_thread:
                sampler_thread.start()
                time.sleep(0.25)
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            begin.record()
            for step in range(steps):
                session.launch()
                history[warmup + step].copy_(session.selected, non_blocking=True)   # 4 bytes a sequence, on the device
            end.record()
            torch.cuda.synchronize()
            runs.append(begin.elapsed_time(end) / steps)
            if sampler_thread:
                clock_record = sampler_thread.stop()
            tokens_of_repeat.append([first] + history.cpu().tolist())
            if profile_steps and repeat == repeats - 1:  # a few more steps inside a profiler range
                session.reserve(profile_steps)
                torch.cuda.profiler.start()
                for _ in range(profile_steps):
                    session.launch()
                torch.cuda.synchronize()
                torch.cuda.profiler.stop()
        finally:
            for slot in slots:
                engine.release(slot)
    ms = statistics.median(runs)
    mean_prompt = sum(len(prompt) for prompt in prompts) / batch
    return {"ms_per_step": ms, "tokens_per_s": batch * 1e3 / ms, "ms_of_repeats": [round(run, 4) for run in runs],
            "kernels_per_step": session.kernels_per_step, "clocks": clock_record,
            "mean_context": mean_prompt + warmup + (steps + 1) / 2, "tokens": tokens_of_repeat[0],
            "repeats_identical": all(tokens == tokens_of_repeat[0] for tokens in tokens_of_repeat)}


def compare_with_plain_steps(engine, sampler, prompts, graph_tokens, steps: int):
    """The same prompts through `Engine.step`, one launch at a time and no graph, fed at every
    step with the tokens the replayed graph selected (so that one differing token does not set
    the two runs apart for good). Returns (tokens compared, tokens that differ, the largest
    distance between the two candidates' logits at a differing token, relative to the largest
    logit of its row). The two paths may split a sequence's keys differently (the graph fixes
    the split for the longest sequence it may hold), so bfloat16 rounding can reorder two logits
    that lie closer than that rounding; a fault would show as a large distance."""
    import torch
    from kidi_b200 import StepBatch
    slots = [engine.acquire() for _ in prompts]
    compared = differing = 0
    largest = 0.0
    try:
        logits = engine.step(StepBatch(slots, prompts, None))
        for step in range(steps + 1):
            chosen = sampler.select(logits).cpu().tolist()
            wanted = graph_tokens[step]
            for row, (mine, theirs) in enumerate(zip(chosen, wanted)):
                compared += 1
                if mine != theirs:
                    differing += 1
                    values = logits[row]
                    distance = float((values[mine] - values[theirs]).abs() / values.abs().max().clamp(min=1.0))
                    largest = max(largest, distance)
            if step < steps:
                logits = engine.step(StepBatch(slots, [[token] for token in wanted], None))
        return compared, differing, largest
    finally:
        for slot in slots:
            engine.release(slot)


def time_prefill(engine, seed: int, repeats: int = 5, profile: bool = False):
    import numpy as np
    import torch
    from kidi_b200 import StepBatch

    generator = np.random.default_rng(seed)
    prompt = generator.integers(0, engine.vocab_size, size=PREFILL_TOKENS).tolist()
    times = []
    for index in range(repeats + 2):
        slot = engine.acquire()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record()
        engine.step(StepBatch([slot], [prompt], None))
        end.record()
        torch.cuda.synchronize()
        engine.release(slot)
        if index >= 2:  # two warm-up runs
            times.append(begin.elapsed_time(end))
    if profile:
        slot = engine.acquire()
        torch.cuda.profiler.start()
        engine.step(StepBatch([slot], [prompt], None))
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        engine.release(slot)
    return statistics.median(times)


def time_end_to_end(engine, prompts, steps: int):
    """Decode tokens a second through `Engine.generate`: host token ids in and out. Returns
    the rate, the statistics and the generated tokens."""
    from kidi_b200.engine.generate import GenerationStats

    batch = len(prompts)
    engine.generate(prompts, max_new_tokens=steps + 1, ignore_eos=True, max_active=batch)   # captures the graph
    stats = GenerationStats()
    found = engine.generate(prompts, max_new_tokens=steps + 1, ignore_eos=True, max_active=batch, stats=stats)
    return batch * stats.decode_steps / (stats.decode_ns / 1e9), stats, found


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=0, help="timed decode steps (default: the model's: 512 / 256)")
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--batch", type=int, default=0, help="sequences of the batch (default: the model's: 8 / 16 / 8)")
    parser.add_argument("--model", default="8b", choices=sorted(MODELS), help="which of the benchmark's shapes")
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0: all)")
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--repeats", type=int, default=REPEATS, help="measured repeats of the decode run (median)")
    parser.add_argument("--skip-points", action="store_true", help="leave out batch 1 / 64 and prefill")
    parser.add_argument("--skip-e2e", action="store_true", help="leave out the end-to-end run (profiling)")
    parser.add_argument("--profile-steps", type=int, default=0,
                        help="run this many extra decode steps inside cudaProfilerStart/Stop")
    parser.add_argument("--profile-prefill", action="store_true",
                        help="run one extra 2,048-token prefill inside cudaProfilerStart/Stop")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference does not build offline: its CMake stops at 'yaml-cpp is missing from "
                          "third_party' (empty submodules), and its Qwen3 is an INT8 bidirectional backbone "
                          "without cache, head or generation"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this library is single-GPU by design (asked for {args.gpus})")
        return 2
    title, shape, default_batch, prompt_lengths, default_steps = MODELS[args.model]
    steps, batch = args.steps or default_steps, args.batch or default_batch
    if steps < 1 or args.warmup < 3 or args.repeats < 1:
        print("bench.py needs --steps >= 1, --warmup >= 3 and --repeats >= 1")
        return 2

    import torch
    from kidi_b200 import Engine
    from kidi_b200.sampling.sampler import Sampler

    config = dict(shape)
    full_layers = config["num_hidden_layers"]
    if args.layers:
        config["num_hidden_layers"] = args.layers
    points_of = () if args.skip_points or args.model != "8b" else (1, 64)
    per_sequence = -(-(prompt_lengths[1] + args.warmup + steps + 2) // 64) * 64
    budget = max(max([batch, *points_of]) * per_sequence, 4096)
    engine = Engine.from_config(config, seed=args.seed, dtype="bfloat16", device="cuda:0", max_tokens=budget)
    sampler = Sampler(args.seed)
    peak = peaks()

    prompts = draw_prompts(engine.vocab_size, batch, prompt_lengths, args.seed)
    main_run = time_decode(engine, sampler, prompts, steps, args.warmup, clocks=True, repeats=args.repeats,
                           profile_steps=args.profile_steps)
    # What vouches for the timed work: the same prompts through plain steps, without the graph.
    compared, mismatches, distance = compare_with_plain_steps(engine, sampler, prompts, main_run["tokens"],
                                                              min(CHECKED_STEPS, args.warmup + steps))
    check = {"repeats": args.repeats, "repeats_identical": main_run["repeats_identical"],
             "tokens_compared_with_plain_steps": compared, "token_mismatches": mismatches,
             "largest_logit_distance_at_a_mismatch": round(distance, 5), "allowed_distance": ROUNDING_DISTANCE,
             "ms_of_repeats": main_run["ms_of_repeats"]}
    if args.skip_e2e:
        from kidi_b200.engine.generate import GenerationStats
        e2e_value, e2e_stats = 0.0, GenerationStats()
    else:
        e2e_value, e2e_stats, generated = time_end_to_end(engine, prompts, steps)
        # The entry point's tokens are the device-timed run's: token n of a sequence is row n of its history.
        check["e2e_token_mismatches"] = sum(
            generated[b][n] != main_run["tokens"][n][b] for b in range(batch)
            for n in range(min(len(generated[b]), len(main_run["tokens"]))))
    if args.profile_prefill:
        time_prefill(engine, args.seed, repeats=1, profile=True)
    points, prefill = {}, None
    for size in points_of:
        run = time_decode(engine, sampler, draw_prompts(engine.vocab_size, size, prompt_lengths, args.seed + size),
                          min(steps, 128), args.warmup, clocks=False, repeats=args.repeats)
        points[f"decode_b{size}"] = round(run["tokens_per_s"], 1)
        check[f"decode_b{size}_repeats_identical"] = run["repeats_identical"]
    if not args.skip_points:
        prefill_ms = time_prefill(engine, args.seed)
        flops = prefill_flops(config, PREFILL_TOKENS)
        prefill = {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "unit": "tokens/s",
                   "tokens": PREFILL_TOKENS, "ms": round(prefill_ms, 3),
                   "frac": round(flops / (prefill_ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4),
                   # `frac` is of the library product's burst rate; the timed prefills run back to back under the
                   # power cap, where that product itself settles at the sustained rate.
                   "frac_of_sustained": round(flops / (prefill_ms / 1e3) /
                                              (peak.get("bf16_tflops_sustained", peak["bf16_tflops"]) * 1e12), 4),
                   "tflops": round(flops / (prefill_ms / 1e3) / 1e12, 1)}

    achieved = decode_bytes(config, batch, main_run["mean_context"]) / (main_run["ms_per_step"] / 1e3) / 1e9
    shortest, longest = prompt_lengths
    prompt_words = f"{shortest}-token prompts" if shortest == longest else f"prompts of {shortest} to {longest} tokens"
    record = {
        "metric": f"decode tokens/s ({title}, bf16, batch {batch}, {prompt_words})",
        "value": round(main_run["tokens_per_s"], 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": steps, "warmup": args.warmup, "ms_per_step": round(main_run["ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0, 0.02) from a seed, uniform token ids", "impl": "ours",
        "config": {
            "model": title, "layers": config["num_hidden_layers"], "layers_of_model": full_layers,
            "hidden_size": config["hidden_size"], "heads": config["num_attention_heads"],
            "kv_heads": config["num_key_value_heads"], "head_dim": config["head_dim"],
            "intermediate_size": config["intermediate_size"], "vocab_size": config["vocab_size"],
            "rope_theta": config["rope_theta"], "rms_norm_eps": config["rms_norm_eps"],
            "tie_word_embeddings": False, "global_batch": batch,
            "prompt_tokens": shortest if shortest == longest else f"uniform in [{shortest}, {longest}]",
            "context_per_sequence": per_sequence if args.model != "8b" else 4096,
            "seq_len": int(main_run["mean_context"]), "parallelism": "single GPU",
            "l2": "no flush: a step reads far more than the 126 MB L2 holds", "peaks": peak["source"],
        },
        "clocks": main_run["clocks"],
        "checked": bool(main_run["repeats_identical"] and distance <= ROUNDING_DISTANCE), "check": check,
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": round(e2e_stats.host_to_device_bytes / max(1, e2e_stats.decode_steps), 1),
                "d2h_bytes_per_step": 4 * batch, "steps": e2e_stats.decode_steps,
                "note": "a step's input tokens are its predecessor's output on the device; the host copies the "
                        "batch's tables up when decoding starts and reads every step's tokens back; decoding "
                        "starts right after the prompts, whose power draw leaves lowered clocks for the first "
                        "twenty steps or so (4.3, then 3.9 ms a step)"},
        "gpu_launches": main_run["kernels_per_step"] * steps,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4), "of": peak["source"]},
    }
    if prefill:
        record["prefill"] = prefill
    if points:
        record["points"] = points
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
