"""Random weights from a configuration and a seed.

The reference has no initialiser ("callers can initialise writable tensors via
state_dict()", ARCHITECTURE.md:873-876; its tests fill constants,
tests/kidi/model/qwen3_test.cpp:42-52). Here every parameter names its own
distribution (`ParamSpec.init`): matrices and tables ~ N(0, std), norm weights ~
1 + N(0, std). Each tensor is drawn from a generator seeded by (seed, tensor name),
so a tensor's values do not depend on which other tensors exist or on their order.

`write_random_model` writes a model folder (config.json, model.safetensors) with the
checkpoint's own unfused names; `random_parameters` fills a model in place on its
device without a file.
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Any, Dict, Iterator, Mapping, Sequence, Tuple

import torch

from ..errors import invalid_argument, io_error
from ..parts.spec import ParamSpec
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    return (int(seed) * 0x9E3779B1 + zlib.crc32(name.encode("utf-8"))) & 0x7FFFFFFFFFFFFFFF


def _draw(name: str, shape: Tuple[int, ...], init: Tuple[str, float], seed: int, dtype: torch.dtype,
          device: torch.device) -> torch.Tensor:
    kind, std = init
    generator = torch.Generator(device=device)
    generator.manual_seed(_tensor_seed(seed, name))
    values = torch.randn(shape, generator=generator, dtype=torch.float32, device=device)
    if kind == "normal":
        values.mul_(std)
    elif kind == "one_plus_normal":
        values.mul_(std).add_(1.0)
    else:
        raise invalid_argument(f"unknown initialiser '{kind}' for tensor '{name}'")
    return values.to(dtype)


def checkpoint_tensors(params: Sequence[Tuple[str, ParamSpec]], seed: int, dtype: torch.dtype,
                       device: torch.device = torch.device("cpu")) -> Iterator[Tuple[str, torch.Tensor]]:
    """Yields (checkpoint name, tensor) for every tensor a file of this model holds:
    fused parameters as their sources, aliased (tied) parameters not at all."""
    for prefix, spec in params:
        if spec.alias_of is not None:
            continue
        if spec.storage != "float":
            raise invalid_argument(f"no random initialiser for {spec.storage} tensor '{prefix + spec.name}'")
        if spec.sources:
            for name, shape in spec.sources:
                yield prefix + name, _draw(prefix + name, tuple(shape), spec.init, seed, dtype, device)
        else:
            yield prefix + spec.name, _draw(prefix + spec.name, tuple(spec.shape), spec.init, seed, dtype, device)


def random_parameters(params: Sequence[Tuple[str, ParamSpec]], seed: int, engine_dtype: torch.dtype,
                      device: torch.device) -> Dict[str, torch.Tensor]:
    """{full parameter name: tensor} drawn on `device`; the values equal those of the
    folder `write_random_model` writes for the same seed when `device` is the CPU."""
    bound: Dict[str, torch.Tensor] = {}
    for prefix, spec in params:
        if spec.alias_of is not None:
            continue
        full = prefix + spec.name
        if spec.sources:
            out = torch.empty(tuple(spec.shape), dtype=engine_dtype, device=device)
            row = 0
            for name, shape in spec.sources:
                out[row:row + shape[0]].copy_(_draw(prefix + name, tuple(shape), spec.init, seed, engine_dtype, device))
                row += shape[0]
            bound[full] = out
        else:
            bound[full] = _draw(full, tuple(spec.shape), spec.init, seed, engine_dtype, device)
    for prefix, spec in params:
        if spec.alias_of is not None:
            bound[prefix + spec.name] = bound[spec.alias_of]
    return bound


def write_random_model(config: Mapping[str, Any], out_dir: str, seed: int = 0,
                       dtype: torch.dtype = torch.bfloat16) -> str:
    """Writes `out_dir/config.json` and `out_dir/model.safetensors` for the
    architecture `config` names, with random weights drawn from `seed`."""
    from ..registry import spec_from_config
    from ..engine.model import declared_parameters

    if dtype not in (torch.bfloat16, torch.float32):
        raise invalid_argument("random weights are written in bfloat16 or float32")
    _, typed, spec = spec_from_config(config)
    params = declared_parameters(spec)
    try:
        os.makedirs(out_dir, exist_ok=True)
        with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as handle:
            values = dict(config)
            values["torch_dtype"] = "bfloat16" if dtype == torch.bfloat16 else "float32"
            json.dump(values, handle, indent=1)
    except OSError as error:
        raise io_error(f"cannot write {out_dir}: {error}") from None
    tensors = dict(checkpoint_tensors(params, seed, dtype))
    path = os.path.join(out_dir, "model.safetensors")
    if os.path.exists(path):
        os.remove(path)
    write_safetensors(path, tensors, metadata={"format": "pt", "seed": str(seed)})
    return out_dir
