"""What every part is: a thing built from a `PartSpec` that declares its tensors,
receives them, and runs on the rows of a step.

Interfaces by role (each is registered with `register_part(role, kind)`):

* norm:          `forward(stream) -> normed`     stream: ResidualStream; applies the pending residual add
* position:      built once per model under a name; mixers look it up in `env.positions`;
                 `on_embeddings(stream, ctx)` may change the embeddings (default: nothing)
* mixer:         `cache_requests() -> [KVRequest | StateRequest]`
                 `forward(x, ctx, views, owns_cache) -> y`   x, y: [rows, hidden] in the engine dtype
* feed_forward:  `forward(x, ctx) -> y`
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


class ResidualStream:
    """The residual stream of a step: `hidden` (float32 [rows, hidden size]) and a
    pending delta that the next norm adds while it normalises, so that the sum is
    formed in 32-bit and the rows are read once."""

    def __init__(self, hidden: torch.Tensor):
        self.hidden = hidden
        self.pending: Optional[torch.Tensor] = None

    def add(self, delta: torch.Tensor) -> None:
        if self.pending is not None:
            raise RuntimeError("a residual delta is pending already; a norm must take it first")
        self.pending = delta

    def take_pending(self) -> Optional[torch.Tensor]:
        delta, self.pending = self.pending, None
        return delta
