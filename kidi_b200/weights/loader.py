"""Binds the tensors of a checkpoint to the parameters a model declares, by name.

The reference checks every name, shape and dtype before it binds anything and
reports unexpected and missing parameters (src/kidi/core/module.cpp:88-107,
src/kidi/model/model.cpp:81-84). This loader does the same in one pass and raises
ONE error that lists every missing tensor, every unexpected tensor and every wrong
shape. A parameter whose own name the file lacks is filled by the first of its
`WeightRule`s whose sources are all there: concatenation along an axis (fused qkv and
gate_up from their parts, src/kidi/model/qwen3.cpp:113-132; one source is a rename), a
slice of a tensor the file stores fused, a transposed matrix, or sources that must be
identical (src/kidi/checkpoint/weights.h:20-31). A parameter with `alias_of` shares the storage of
its target when the file does not carry it (tied embeddings; the reference's
`tie_parameter`, src/kidi/core/module.cpp:60-69,132-147) and must equal the target
when it does.

dtype policy: a tensor the file stores in bfloat16 stays bfloat16 and one it stores
in 32-bit stays 32-bit (float16 widens to 32-bit, which holds it exactly); integer
tables become int32. A float32 engine widens everything to float32 (exact). A bfloat16
engine warns when matrices stay 32-bit, since their products then run on the 32-bit
kernel, and rounds them to bfloat16 instead when asked to (`cast_matrices`).
"""
from __future__ import annotations

import json
import os
import re
import warnings
from typing import Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

import torch

from ..errors import invalid_argument, invalid_manifest, io_error
from ..parts.spec import ParamSpec, WeightRule, renamed
from .safetensors_io import SafetensorsFile

WEIGHTS_FILE = "model.safetensors"
INDEX_FILE = "model.safetensors.index.json"

_FLOAT_TYPES = (torch.bfloat16, torch.float32, torch.float16, torch.float64)
_INT_TYPES = (torch.int32, torch.int64, torch.int8, torch.uint8)


class Checkpoint:
    """The tensors of a model folder: one model.safetensors, or the shards an index names."""

    def __init__(self, model_dir: str):
        self.files: List[SafetensorsFile] = []
        self._where: Dict[str, SafetensorsFile] = {}
        single = os.path.join(model_dir, WEIGHTS_FILE)
        index = os.path.join(model_dir, INDEX_FILE)
        if os.path.exists(single):
            paths = [single]
        elif os.path.exists(index):
            try:
                with open(index, "r", encoding="utf-8") as handle:
                    weight_map = json.load(handle)["weight_map"]
            except (OSError, KeyError, json.JSONDecodeError) as error:
                raise invalid_manifest(f"{index}: {error}") from None
            names = sorted(set(weight_map.values()))
            for name in names:
                if os.path.isabs(name) or ".." in name.split("/"):
                    raise invalid_manifest(f"{index}: shard path '{name}' leaves the model folder")
            paths = [os.path.join(model_dir, name) for name in names]
        else:
            raise io_error(f"no {WEIGHTS_FILE} (or {INDEX_FILE}) in {model_dir}")
        for path in paths:
            file = SafetensorsFile(path)
            self.files.append(file)
            for name in file.names():
                if name in self._where:
                    raise invalid_manifest(f"tensor '{name}' occurs in two shards")
                self._where[name] = file

    def names(self) -> Iterable[str]:
        return self._where.keys()

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._where[name].shape(name)

    def dtype(self, name: str) -> torch.dtype:
        return self._where[name].dtype(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self._where[name].tensor(name)

    def close(self) -> None:
        for file in self.files:
            file.close()


class TensorDict:
    """The same reading interface over tensors already in memory (tests, random weights)."""

    def __init__(self, tensors: Mapping[str, torch.Tensor]):
        self._tensors = dict(tensors)

    def names(self):
        return self._tensors.keys()

    def __contains__(self, name):
        return name in self._tensors

    def shape(self, name):
        return tuple(self._tensors[name].shape)

    def dtype(self, name):
        return self._tensors[name].dtype

    def tensor(self, name):
        return self._tensors[name]

    def close(self):
        pass


def _stored_dtype(file_dtype: torch.dtype, storage: str, engine_dtype: torch.dtype) -> Optional[torch.dtype]:
    if storage == "int32":
        return torch.int32 if file_dtype in _INT_TYPES else None
    if file_dtype not in _FLOAT_TYPES:
        return None
    if engine_dtype == torch.float32:
        return torch.float32
    return torch.bfloat16 if file_dtype == torch.bfloat16 else torch.float32


def _assemble(rule: WeightRule, names: Sequence[str], source, target: torch.dtype, device: torch.device,
              full: str) -> torch.Tensor:
    """The parameter a rule makes of its sources, on `device` in `target`."""
    fetch = lambda name: source.tensor(name).to(device=device, dtype=target)
    if rule.op == "concat":
        if len(names) == 1:
            return fetch(names[0]).contiguous()
        out = torch.empty(rule.result_shape(), dtype=target, device=device)
        cursor = 0
        for name, (_, shape) in zip(names, rule.sources):
            out.narrow(rule.axis, cursor, shape[rule.axis]).copy_(fetch(name))
            cursor += shape[rule.axis]
        return out
    if rule.op == "split":
        return source.tensor(names[0]).narrow(rule.axis, rule.start, rule.length).to(
            device=device, dtype=target).contiguous()
    if rule.op == "transpose":
        return fetch(names[0]).t().contiguous()
    if rule.op == "identical":
        first = fetch(names[0]).contiguous()
        for name in names[1:]:
            if not torch.equal(fetch(name), first):
                raise invalid_manifest(f"'{full}': '{name}' must hold the same values as '{names[0]}'")
        return first
    raise invalid_argument(f"unknown weight rule '{rule.op}' for '{full}'")


def bind_parameters(params: Sequence[Tuple[str, ParamSpec]], source, *, engine_dtype: torch.dtype,
                    device: torch.device, ignored: Sequence[str] = (),
                    cast_matrices: bool = False) -> Dict[str, torch.Tensor]:
    """Returns {full parameter name: tensor on `device`} or raises one error that
    lists everything that does not fit. `params` pairs a name prefix with each spec.
    With `cast_matrices`, a bfloat16 engine rounds matrices that the file stores wider
    (float32, float16) to bfloat16; without, they stay 32-bit, their products run on the
    32-bit kernel, and a warning says so."""
    missing: List[str] = []
    wrong: List[str] = []
    plans = []  # (full name, rule or None for an alias, [full source names], spec)
    consumed = set()
    declared = {prefix + spec.name: spec for prefix, spec in params}
    for prefix, spec in params:
        full = prefix + spec.name
        alternatives = spec.alternatives()
        chosen = None
        for rule in (renamed(spec.name, spec.shape), *alternatives):
            if rule.op == "split" and not (0 <= rule.start and rule.length > 0
                                           and rule.start + rule.length <= rule.sources[0][1][rule.axis]):
                raise invalid_argument(f"'{full}': a split rule reaches outside its source")
            if tuple(rule.result_shape()) != tuple(spec.shape):
                raise invalid_argument(f"'{full}': a weight rule makes shape {list(rule.result_shape())}, "
                                       f"the parameter has {list(spec.shape)}")
            names = [prefix + name for name, _ in rule.sources]
            if all(name in source for name in names):
                chosen = (rule, names)
                break
        if chosen is not None:
            plans.append((full, chosen[0], chosen[1], spec))
            consumed.update(chosen[1])
            continue
        absent: List[str] = []
        for rule in alternatives:
            names = [prefix + name for name, _ in rule.sources]
            present = [name for name in names if name in source]
            consumed.update(present)  # expected, though incomplete
            if present and not absent:
                absent = [name for name in names if name not in source]
        if spec.alias_of is not None:
            if spec.alias_of not in declared:
                wrong.append(f"{full}: tied to '{spec.alias_of}', which the model does not declare")
            plans.append((full, None, [], spec))
        elif absent:
            missing.extend(absent)
        elif alternatives:
            missing.extend(prefix + name for name, _ in alternatives[0].sources)
        else:
            missing.append(full)
    patterns = [re.compile(pattern) for pattern in ignored]
    unexpected = sorted(name for name in source.names()
                        if name not in consumed and not any(p.search(name) for p in patterns))
    for full, rule, names, spec in plans:
        if rule is None:
            continue
        for name, (_, shape) in zip(names, rule.sources):
            found = tuple(source.shape(name))
            if found != tuple(shape):
                wrong.append(f"{name}: shape {list(found)} in the file, {list(shape)} expected")
            if _stored_dtype(source.dtype(name), spec.storage, engine_dtype) is None:
                wrong.append(f"{name}: dtype {source.dtype(name)} cannot fill a {spec.storage} parameter")
    missing = sorted(set(missing))
    if missing or unexpected or wrong:
        lines = ["the checkpoint does not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes or types ({len(wrong)}): " + "; ".join(sorted(set(wrong))))
        raise invalid_manifest("\n".join(lines))

    bound: Dict[str, torch.Tensor] = {}
    wide: List[str] = []
    for full, rule, names, spec in plans:
        if rule is None:
            continue
        target = _stored_dtype(source.dtype(names[0]), spec.storage, engine_dtype)
        for name in names[1:]:
            if _stored_dtype(source.dtype(name), spec.storage, engine_dtype) != target:
                target = torch.float32
        if engine_dtype == torch.bfloat16 and target == torch.float32 and len(spec.shape) >= 2:
            if cast_matrices:
                target = torch.bfloat16
            else:
                wide.append(full)
        bound[full] = _assemble(rule, names, source, target, device, full)
    if wide:
        warnings.warn(
            f"{len(wide)} matrices (the first: {wide[0]}) are stored wider than bfloat16 and stay 32-bit: their "
            f"products run on the 32-bit kernel, far slower than the bfloat16 ones; load with cast_weights=True "
            f"(command line: --cast-weights) to round them to bfloat16", stacklevel=2)
    for full, rule, names, spec in plans:
        if rule is None:
            bound[full] = bound[spec.alias_of]
        elif spec.alias_of is not None:
            target = bound[spec.alias_of]
            if bound[full].shape != target.shape or not torch.equal(bound[full].to(target.dtype), target):
                raise invalid_manifest(f"'{full}' is tied to '{spec.alias_of}' but the file holds different values")
            bound[full] = target
    return bound
