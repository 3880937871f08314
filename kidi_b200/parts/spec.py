"""Data that describes a model before any tensor exists.

A model is a `ModelSpec`: an embedding, named position encodings, a list of layers,
a schedule (the order in which layers run), a final norm and an output head. Each
of these is a `PartSpec`: the registry key of a part, the sizes and constants that
part takes as parameters, and the prefix of its tensor names. An architecture is a
function from its typed configuration to a `ModelSpec`; nothing below that function
knows which architecture it is in.

The reference keeps the same separation with constructor parameters
(`Qwen3Shape`, src/kidi/layers/qwen3.h:7-15) and a layer-to-cache map
(src/kidi/model/gemma4.cpp:149-155).
"""
from __future__ import annotations

import dataclasses
from typing import Any, Mapping, Optional, Sequence, Tuple


@dataclasses.dataclass(frozen=True)
class PartSpec:
    kind: str
    params: Mapping[str, Any] = dataclasses.field(default_factory=dict)
    prefix: str = ""

    def param(self, key: str, default: Any = dataclasses.MISSING) -> Any:
        if key in self.params:
            return self.params[key]
        if default is dataclasses.MISSING:
            raise KeyError(f"part '{self.kind}' needs parameter '{key}'")
        return default


@dataclasses.dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (how norms, mixer and feed-forward are wired around
    the residual stream) and the parts it arranges, by role."""

    arrangement: PartSpec
    parts: Mapping[str, PartSpec]


@dataclasses.dataclass(frozen=True)
class ScheduleEntry:
    """One position in the run order. `layer` indexes `ModelSpec.layers` and may
    occur at several positions (shared weights; each position has a cache of its
    own). `cache_from` names an EARLIER position whose cache this one reads instead
    of keeping one."""

    layer: int
    cache_from: Optional[int] = None


@dataclasses.dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    positions: Mapping[str, PartSpec]
    layers: Sequence[LayerSpec]
    schedule: Sequence[ScheduleEntry]
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: Tuple[int, ...] = ()
    ignored_tensors: Tuple[str, ...] = ()  # regular expressions of tensor names a file may carry unused


@dataclasses.dataclass(frozen=True)
class WeightRule:
    """One way to fill a parameter from tensors that a checkpoint carries under other names
    or in another layout. The reference states such mappings as data too
    (`StateMappingSpec` with CONCAT, IDENTICAL and IGNORE and a regular-expression rename,
    src/kidi/checkpoint/weights.h:20-31, used in src/kidi/model/qwen3.cpp:113-132).

    `sources` are (name relative to the part's prefix, shape in the file) pairs.
    * "concat":    the sources joined along `axis`, in order (one source: a rename);
    * "split":     rows [start, start + length) along `axis` of the one source (a tensor the
                   file stores fused and several parameters share);
    * "transpose": the one source, a matrix, with its axes swapped;
    * "identical": every source must hold the same values; the parameter takes the first.
    Tensors that a file may carry unused are named by `Part.ignored_tensors` and
    `ModelSpec.ignored_tensors`."""

    op: str
    sources: Tuple[Tuple[str, Tuple[int, ...]], ...]
    axis: int = 0
    start: int = 0
    length: int = 0

    def result_shape(self) -> Tuple[int, ...]:
        first = tuple(self.sources[0][1])
        if self.op == "concat":
            joined = list(first)
            joined[self.axis] = sum(shape[self.axis] for _, shape in self.sources)
            return tuple(joined)
        if self.op == "split":
            cut = list(first)
            cut[self.axis] = self.length
            return tuple(cut)
        if self.op == "transpose":
            return (first[1], first[0])
        if self.op == "identical":
            return first
        raise ValueError(f"unknown weight rule '{self.op}'")


def renamed(name: str, shape) -> WeightRule:
    return WeightRule("concat", ((name, tuple(shape)),))


def concatenated(sources, axis: int = 0) -> WeightRule:
    return WeightRule("concat", tuple((name, tuple(shape)) for name, shape in sources), axis=axis)


def split_from(name: str, shape, axis: int, start: int, length: int) -> WeightRule:
    return WeightRule("split", ((name, tuple(shape)),), axis=axis, start=start, length=length)


def transposed(name: str, shape) -> WeightRule:
    return WeightRule("transpose", ((name, tuple(shape)),))


def identical(sources) -> WeightRule:
    return WeightRule("identical", tuple((name, tuple(shape)) for name, shape in sources))


@dataclasses.dataclass(frozen=True)
class ParamSpec:
    """One tensor a part owns.

    `name` is relative to the part's prefix. When a checkpoint does not carry that name,
    `rules` are tried in order (the first whose sources are all present fills the
    parameter). `sources`, if given, is shorthand for the first such rule: (name, shape)
    pairs concatenated on axis 0 in order, which is the reference's q/k/v -> qkv and
    gate/up -> gate_up rule (src/kidi/model/qwen3.cpp:113-132).
    `init` names the random-weights distribution: ("normal", std) or
    ("one_plus_normal", std). `storage` is "float" (bfloat16, or 32-bit when the
    file stores 32-bit) or "int32".
    """

    name: str
    shape: Tuple[int, ...]
    init: Tuple[str, float] = ("normal", 0.02)
    sources: Optional[Tuple[Tuple[str, Tuple[int, ...]], ...]] = None
    storage: str = "float"
    alias_of: Optional[str] = None  # full name of a tensor this one shares storage with when absent
    rules: Tuple[WeightRule, ...] = ()

    def alternatives(self) -> Tuple[WeightRule, ...]:
        """The rules that can fill this parameter when its own name is absent."""
        first = (concatenated(self.sources),) if self.sources else ()
        return first + tuple(self.rules)
