"""The command line, in the manner of the reference's `kidi` program.

    kidi_b200 generate -m MODEL [-i FILE] [-o FILE] [--max-new-tokens N] [--context-size N]
                       [--prefill-chunk-size N] [--ignore-eos] [--cache-tokens N] [--max-active N]
                       [--precision checkpoint|bf16|fp32] [--cast-weights] [--backend auto|cuda[:INDEX]] [--profile]
                       [--temperature T] [--seed S]
    kidi_b200 inspect -m MODEL
    kidi_b200 random-model --config CONFIG.json --seed S -o MODEL [--precision bf16|fp32]

Option names, defaults and meanings are the reference's where it has them
(src/kidi/cli/main.cpp:835-856,905-958,995-1006): `-m/--model`, `--backend`, `--profile`,
`--max-new-tokens 0`, `--context-size 0`, `--prefill-chunk-size`, `--ignore-eos`,
`--cache-tokens 16384`, `--max-active` (default 4), `--queue-size 64`, `--precision`,
`--kv-cache-precision`, `-i/--in -`, `-o/--out -`. `generate` reads one JSON object a line
and writes one a line (src/kidi/cli/main.cpp:205-244,369-391). The reference's requests
carry chat `messages` and need its tokenizer; this library works on token ids, so a
request is `{"token_ids": [...], "id"?, "max_tokens"?}` and a record is
`{"request_id", "id", "token_ids", "decoder_steps", "finish"}` (with `--profile` also the
timing fields of src/kidi/cli/main.cpp:376-390). Results go to the output, diagnostics to
stderr; exit codes are 0, 1 for a runtime fault and 2 for a usage fault
(src/kidi/cli/main.cpp:1028-1035). `--temperature`, `--seed` and `random-model` are this
library's own.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List, Optional

from .errors import KidiError, invalid_argument


class _UsageError(Exception):
    pass


class _Parser(argparse.ArgumentParser):
    def error(self, message):  # argparse would exit the interpreter; the entry point returns a code
        raise _UsageError(f"{self.format_usage()}{self.prog}: error: {message}")


def build_parser() -> argparse.ArgumentParser:
    parser = _Parser(prog="kidi_b200", description="Qwen3 generation on one B200, in the manner of kidi.")
    commands = parser.add_subparsers(dest="command", metavar="COMMAND", parser_class=_Parser)
    commands.required = True

    generate = commands.add_parser("generate", help="generate token ids for JSONL requests")
    inspect = commands.add_parser("inspect", help="print what a model folder holds")
    random_model = commands.add_parser("random-model", help="write a model folder with random weights")

    for command in (generate, inspect):
        command.add_argument("-m", "--model", required=True, metavar="MODEL",
                             help="local directory with config.json and model.safetensors")
    generate.add_argument("--backend", default="auto", help="auto or cuda[:INDEX]")
    generate.add_argument("--profile", action="store_true")
    generate.add_argument("--cache-tokens", dest="cache_tokens", type=int, default=16384,
                          help="budget for reserved context tokens")
    generate.add_argument("--max-new-tokens", dest="max_new_tokens", type=int, default=0)
    generate.add_argument("--context-size", dest="context_size", type=int, default=0)
    generate.add_argument("--prefill-chunk-size", dest="prefill_chunk_size", type=int, default=0,
                          help="prompt tokens per sequence and step (0: whole prompts)")
    generate.add_argument("--ignore-eos", dest="ignore_eos", action="store_true")
    generate.add_argument("--precision", default="checkpoint", choices=["checkpoint", "bf16", "fp32"],
                          help="compute policy; checkpoint follows the dtype of the weights file")
    generate.add_argument("--cast-weights", dest="cast_weights", action="store_true",
                          help="round matrices stored wider than bfloat16 to bfloat16 (implied by --precision bf16)")
    generate.add_argument("--kv-cache-precision", dest="kv_cache_precision", default="auto",
                          choices=["auto", "fp32", "bf16"], help="auto: the compute precision")
    generate.add_argument("--max-active", dest="max_active", type=int, default=None, metavar="N",
                          help="active concurrent requests (default: 4)")
    generate.add_argument("--queue-size", dest="queue_size", type=int, default=64)
    generate.add_argument("--temperature", type=float, default=0.0, help="0: greedy")
    generate.add_argument("--seed", type=int, default=0)
    generate.add_argument("-i", "--in", dest="input", default="-", metavar="FILE", help="input file, or '-' for stdin")
    generate.add_argument("-o", "--out", dest="output", default="-", metavar="FILE",
                          help="output file, or '-' for stdout")

    random_model.add_argument("--config", required=True, metavar="JSON", help="a config.json to build from")
    random_model.add_argument("--seed", type=int, default=0)
    random_model.add_argument("--precision", default="bf16", choices=["bf16", "fp32"])
    random_model.add_argument("-o", "--out", dest="output", required=True, metavar="MODEL")
    return parser


def _log(message: str) -> None:
    print(f"kidi_b200: {message}", file=sys.stderr, flush=True)


def _device(backend: str) -> str:
    if backend == "auto" or backend == "cuda":
        return "cuda:0"
    if backend.startswith("cuda:") and backend[5:].isdigit():
        return backend
    raise invalid_argument(f"backend '{backend}' is not available here (auto or cuda[:INDEX])")


def _read_requests(stream) -> List[dict]:
    requests = []
    for number, line in enumerate(stream, 1):
        line = line.strip()
        if not line:
            continue
        try:
            request = json.loads(line)
        except json.JSONDecodeError as error:
            raise invalid_argument(f"input line {number} is not JSON: {error}") from None
        if not isinstance(request, dict) or not isinstance(request.get("token_ids"), list) or not request["token_ids"]:
            raise invalid_argument(f"input line {number}: expected an object with a nonempty token_ids array")
        for key in request:
            if key not in ("token_ids", "id", "max_tokens"):
                raise invalid_argument(f"input line {number}: unsupported request field: {key}")
        if not all(isinstance(token, int) and not isinstance(token, bool) for token in request["token_ids"]):
            raise invalid_argument(f"input line {number}: token_ids must be integers")
        if "id" in request and not isinstance(request["id"], (str, int)):
            raise invalid_argument(f"input line {number}: id must be a string or integer")
        limit = request.get("max_tokens")
        if limit is not None and (not isinstance(limit, int) or isinstance(limit, bool) or limit <= 0 or limit > 2**31 - 1):
            raise invalid_argument(f"input line {number}: max_tokens must be a positive integer within int32 bounds")
        requests.append(request)
    return requests


def _generate(args) -> int:
    import torch
    from .config.reader import read_config_json
    from .engine.engine import Engine
    from .engine.generate import DEFAULT_MAX_ACTIVE, GenerationStats
    from .weights.loader import Checkpoint

    started = time.perf_counter_ns()
    device = _device(args.backend)
    precision = args.precision
    if precision == "checkpoint":  # the dtype of a probe tensor of the file, as the reference does
        read_config_json(args.model)
        checkpoint = Checkpoint(args.model)
        try:
            kinds = {checkpoint.dtype(name) for name in checkpoint.names() if len(checkpoint.shape(name)) == 2}
        finally:
            checkpoint.close()
        precision = "fp32" if kinds and kinds <= {torch.float32, torch.float64} else "bf16"
    if args.kv_cache_precision not in ("auto", precision):
        raise invalid_argument("the cache is kept in the compute precision (--kv-cache-precision auto)")
    if args.cache_tokens <= 0 or args.queue_size <= 0:
        raise invalid_argument("--cache-tokens and --queue-size must be positive")
    max_active = args.max_active if args.max_active is not None else DEFAULT_MAX_ACTIVE
    # An explicit --precision bf16 asks for bfloat16 products: matrices a file stores wider are
    # rounded at load. With "checkpoint" every tensor keeps the width the file stores it in.
    engine = Engine.load(args.model, dtype=precision, device=device, max_tokens=args.cache_tokens,
                         cast_weights=args.precision == "bf16" or args.cast_weights)
    load_ns = time.perf_counter_ns() - started

    source = sys.stdin if args.input == "-" else open(args.input, "r", encoding="utf-8")
    try:
        requests = _read_requests(source)
    finally:
        if source is not sys.stdin:
            source.close()
    sink = sys.stdout if args.output == "-" else open(args.output, "w", encoding="utf-8")
    try:
        stats = GenerationStats()
        results = engine.generate(
            [request["token_ids"] for request in requests], max_new_tokens=args.max_new_tokens,
            temperature=args.temperature, seed=args.seed, ignore_eos=args.ignore_eos, max_active=max_active,
            context_size=args.context_size, prefill_chunk_size=args.prefill_chunk_size,
            max_tokens=[request.get("max_tokens") for request in requests], stats=stats, detailed=True)
        for index, (request, generation) in enumerate(zip(requests, results)):
            record = {"request_id": index, "id": request.get("id"), "token_ids": generation.token_ids,
                      "decoder_steps": generation.decoder_steps, "finish": generation.finish_reason}
            if args.profile:
                record["prompt_tokens"] = len(request["token_ids"])
                record["decode_tokens"] = len(generation.token_ids)
            sink.write(json.dumps(record) + "\n")
        sink.flush()
    finally:
        if sink is not sys.stdout:
            sink.close()
    if args.profile:
        memory = engine.memory()
        print(f"kidi_serving|requests={len(requests)}|max_active={max_active}|backend=cuda|device={device}"
              f"|load_ns={load_ns}|precision={precision}|cache_tokens={engine.cache.max_tokens}"
              f"|weight_bytes={memory['weight_bytes']}|cache_bytes={memory['cache_bytes']}"
              f"|batches={stats.batches}|prompt_tokens={stats.prompt_tokens}|decode_tokens={stats.generated_tokens}"
              f"|ttft_ns={stats.time_to_first_token_ns}|prefill_ns={stats.prefill_ns}|decode_ns={stats.decode_ns}"
              f"|generation_ns={stats.generation_ns}", file=sys.stderr, flush=True)
    return 0


def _inspect(args) -> int:
    from .config.reader import read_config_json
    from .engine.model import declared_parameters
    from .registry import spec_from_config
    from .weights.loader import Checkpoint

    entry, typed, spec = spec_from_config(read_config_json(args.model))
    print(f"architecture: {entry.name}")
    print(f"layers: {len(spec.layers)} (run order: {len(spec.schedule)} entries)")
    print(f"hidden: {spec.hidden_size}  vocabulary: {spec.vocab_size}  positions: {spec.max_positions}")
    for key, value in sorted(vars(typed).items()) if hasattr(typed, "__dict__") else []:
        print(f"config.{key}: {value}")
    checkpoint = Checkpoint(args.model)
    try:
        names = list(checkpoint.names())
        total = sum(int(__import__("math").prod(checkpoint.shape(name))) for name in names)
        print(f"tensors: {len(names)}  parameters: {total}")
    finally:
        checkpoint.close()
    print(f"declared parameters: {len(declared_parameters(spec))}")
    return 0


def _random_model(args) -> int:
    import torch
    from .weights.random_init import write_random_model
    try:
        with open(args.config, "r", encoding="utf-8") as handle:
            config = json.load(handle)
    except OSError as error:
        _log(f"cannot read {args.config}: {error}")
        return 1
    write_random_model(config, args.output, seed=args.seed,
                       dtype=torch.bfloat16 if args.precision == "bf16" else torch.float32)
    _log(f"wrote {args.output}")
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    """Runs the command line on `argv` (default: the process arguments) and returns
    the exit code; it never exits the interpreter."""
    argv = list(sys.argv[1:] if argv is None else argv)
    parser = build_parser()
    try:
        args = parser.parse_args(argv)
    except _UsageError as error:
        print(error, file=sys.stderr)
        return 2
    except SystemExit as exit_request:  # --help
        return int(exit_request.code or 0)
    try:
        if args.command == "generate":
            return _generate(args)
        if args.command == "inspect":
            return _inspect(args)
        return _random_model(args)
    except KidiError as error:
        _log(error.message)
        return 1
    except (OSError, ValueError, RuntimeError) as error:
        _log(str(error))
        return 1
