"""What every part is: a thing built from a `PartSpec` that declares its tensors,
receives them, and runs on the rows of a step.

Interfaces by role (each is registered with `register_part(role, kind)`):

* norm:          `forward(stream) -> normed`     stream: ResidualStream; applies the pending residual add
* position:      built once per model under a name; mixers look it up in `env.positions`;
                 `on_embeddings(stream, ctx)` may change the embeddings (default: nothing)
* mixer:         `cache_requests() -> [KVRequest | StateRequest]`
                 `forward(x, ctx, views, owns_cache) -> y`   x, y: [rows, hidden] in the engine dtype
* feed_forward:  `forward(x, ctx) -> y`
                 (both optionally: class attribute `accepts_row_scaled = True`: x may be a `RowScaled`;
                 `takes_sink = True`: `forward(..., sink=ResidualSink)` may return None after adding y
                 to the residual stream itself)
* arrangement:   `__init__(spec, env, parts)`; `forward(stream, ctx, views, owns_cache)`
* embedding:     `forward(tokens, ctx) -> float32 [rows, hidden]`
* head:          `forward(x, ctx) -> float32 [rows, vocab]`

No part knows which model it is in: sizes and constants arrive in `spec.params`, tensor
names under `spec.prefix`.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .spec import ParamSpec, PartSpec


@dataclasses.dataclass
class BuildEnv:
    """What parts are built against."""

    dtype: torch.dtype                 # element type of activations, cache and (bfloat16-stored) weights
    device: torch.device
    max_positions: int
    positions: Dict[str, object] = dataclasses.field(default_factory=dict)


class Part:
    role = "part"
    kind = "part"

    def __init__(self, spec: PartSpec, env: BuildEnv):
        self.spec = spec
        self.env = env
        self.prefix = spec.prefix

    # --- tensors
    def parameter_specs(self) -> List[ParamSpec]:
        """The tensors this part owns, named relative to its prefix."""
        return []

    def ignored_tensors(self) -> Sequence[str]:
        """Regular expressions, relative to the part's prefix, of tensors a checkpoint may
        carry for this part without the part using them (the reference's IGNORE mapping,
        src/kidi/checkpoint/weights.h:20-24)."""
        return ()

    def children(self) -> Sequence["Part"]:
        return ()

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receives {relative name: tensor} for the tensors of `parameter_specs`."""
        for name, tensor in tensors.items():
            setattr(self, "_" + name.replace(".", "_"), tensor)

    # --- cache
    def cache_requests(self) -> list:
        return []

    # --- captured steps
    def launch_signature(self, rows: int, longest: int) -> tuple:
        """What a captured decode step of `rows` sequences of at most `longest` tokens would
        freeze of this part's launch choices (grid shapes that depend on the sequence length,
        say). Two steps with equal signatures can replay one captured graph. Default: the
        signatures of the part's children."""
        return tuple(child.launch_signature(rows, longest) for child in self.children())


def all_parameters(part: Part) -> List[Tuple[str, ParamSpec]]:
    """(prefix, spec) of the part and of its children, depth first."""
    found = [(part.prefix, spec) for spec in part.parameter_specs()]
    for child in part.children():
        found.extend(all_parameters(child))
    return found


def bind_all(part: Part, bound: Dict[str, torch.Tensor]) -> None:
    own = {spec.name: bound[part.prefix + spec.name] for spec in part.parameter_specs()}
    if own:
        part.bind(own)
    for child in part.children():
        bind_all(child, bound)


class RowScaled:
    """Normalised rows kept in two pieces, so that no kernel of its own has to normalise them:
    `values` [rows, width] (bfloat16: the residual times the norm's weight, not yet divided by
    the row's root mean square) and `parts` [rows, count] (float32: parts of each row's sum of
    squares). Row r of the normalised matrix is values[r] / sqrt(sum(parts[r]) / width + eps).
    A product of such rows with a weight matrix applies the factor to its result
    (`Linear.forward`); `plain()` makes an ordinary matrix for any other consumer. Only parts
    that set `accepts_row_scaled` are ever handed one."""

    def __init__(self, values: torch.Tensor, parts: torch.Tensor, width: int, eps: float):
        self.values, self.parts, self.width, self.eps = values, parts, int(width), float(eps)

    @property
    def shape(self):
        return self.values.shape

    @property
    def dtype(self):
        return self.values.dtype

    @property
    def factors(self):
        return (self.parts, self.width, self.eps)

    def plain(self) -> torch.Tensor:
        from ..kernels import ops
        return ops.apply_row_factors(self.values, self.parts, self.width, self.eps)


def plain_rows(x) -> torch.Tensor:
    """x as an ordinary matrix, whatever it was handed as."""
    return x.plain() if isinstance(x, RowScaled) else x


class ResidualSink:
    """An offer to the product that ends a mixer or a feed-forward: instead of returning its
    result (which the arrangement would add to the residual stream, and the next norm would
    read again), it may add the result to the stream itself and leave the rows for `norm`
    prepared (`ResidualStream.prepared`). A product that cannot do so ignores the offer and
    returns its result as ever. `norm` is the part that reads the stream next and takes such
    rows (`norm.prepared_weight()` is its weight vector)."""

    def __init__(self, stream: "ResidualStream", norm: "Part"):
        self.stream, self.norm = stream, norm


class ResidualStream:
    """The residual stream of a step: `hidden` (float32 [rows, hidden size]) and a
    pending delta that the next norm adds while it normalises, so that the sum is
    formed in 32-bit and the rows are read once. A product that took a `ResidualSink` has
    added its result already and left `prepared` = (norm, values, parts) for that norm."""

    def __init__(self, hidden: torch.Tensor):
        self.hidden = hidden
        self.pending: Optional[torch.Tensor] = None
        self.prepared = None

    def add(self, delta: Optional[torch.Tensor]) -> None:
        """`delta` None: the part that made it has added it through a sink already."""
        if delta is None:
            return
        if self.pending is not None:
            raise RuntimeError("a residual delta is pending already; a norm must take it first")
        self.pending = delta
        self.prepared = None          # rows prepared before this delta are no longer the stream's

    def take_pending(self) -> Optional[torch.Tensor]:
        delta, self.pending = self.pending, None
        return delta

    def take_prepared(self, norm) -> Optional[tuple]:
        """(values, parts) if the stream's rows were prepared for `norm`, once."""
        prepared, self.prepared = self.prepared, None
        if prepared is not None and prepared[0] is norm and self.pending is None:
            return prepared[1], prepared[2]
        return None
