"""A causal language model put together from a `ModelSpec`.

The model owns an embedding, named position encodings, layers (each an arrangement of
a mixer, a feed-forward and norms), a schedule, a final norm and a head; it knows
nothing about any architecture. Its forward pass is the reference's order of
operations (src/kidi/model/qwen3.cpp:181-204: embeddings, every block, final norm)
followed by the head at the wanted rows, over the packed rows of one step.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import torch

from ..errors import invalid_argument
from ..parts import registry as part_registry
from ..parts.base import BuildEnv, Part, ResidualStream, all_parameters, bind_all
from ..parts.spec import ModelSpec, ParamSpec

# Importing the built-in parts registers them.
from ..parts import arrangement as _arrangement  # noqa: F401
from ..parts import attention as _attention  # noqa: F401
from ..parts import embedding as _embedding  # noqa: F401
from ..parts import feed_forward as _feed_forward  # noqa: F401
from ..parts import norm as _norm  # noqa: F401
from ..parts import position as _position  # noqa: F401


class CausalLM:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device):
        if dtype not in (torch.bfloat16, torch.float32):
            raise invalid_argument("the engine runs in bfloat16 or float32")
        self.spec = spec
        self.env = BuildEnv(dtype=dtype, device=torch.device(device), max_positions=spec.max_positions)
        for name, position in spec.positions.items():
            self.env.positions[name] = part_registry.build_part("position", position, self.env)
        self.embedding = part_registry.build_part("embedding", spec.embedding, self.env)
        self.layers: List[Part] = []
        for layer in spec.layers:
            arrangement = part_registry.part_class("arrangement", layer.arrangement.kind)
            roles = arrangement.ROLES
            missing = [role for role in roles if role not in layer.parts]
            if missing:
                raise invalid_argument(f"arrangement '{layer.arrangement.kind}' lacks parts: {', '.join(missing)}")
            parts = {role: part_registry.build_part(roles[role], layer.parts[role], self.env) for role in roles}
            self.layers.append(arrangement(layer.arrangement, self.env, parts))
        self.final_norm = part_registry.build_part("norm", spec.final_norm, self.env)
        self.head = part_registry.build_part("head", spec.head, self.env)
        self.schedule = list(spec.schedule)
        for index, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise invalid_argument(f"the schedule names layer {entry.layer}, which does not exist")
            if entry.cache_from is not None and not 0 <= entry.cache_from < index:
                raise invalid_argument("a schedule entry may read the cache of an earlier entry only")
        self.loaded = False

    # ------------------------------------------------------------------ tensors
    def _top_parts(self) -> Sequence[Part]:
        return [self.embedding, *self.env.positions.values(), *self.layers, self.final_norm, self.head]

    def parameters(self) -> List[Tuple[str, ParamSpec]]:
        found: List[Tuple[str, ParamSpec]] = []
        for part in self._top_parts():
            found.extend(all_parameters(part))
        names = [prefix + spec.name for prefix, spec in found]
        if len(set(names)) != len(names):
            raise invalid_argument("two parts declare the same tensor name")
        return found

    def ignored_tensors(self) -> List[str]:
        """Regular expressions of tensor names a checkpoint may carry unused: the model's
        own and those its parts name relative to their prefixes."""
        import re

        def collect(part: Part) -> List[str]:
            found = ["^" + re.escape(part.prefix) + pattern.lstrip("^") for pattern in part.ignored_tensors()]
            for child in part.children():
                found.extend(collect(child))
            return found

        patterns = list(self.spec.ignored_tensors)
        for part in self._top_parts():
            patterns.extend(collect(part))
        return patterns

    def bind(self, bound: Dict[str, torch.Tensor]) -> None:
        for part in self._top_parts():
            bind_all(part, bound)
        self.weight_bytes = sum(t.numel() * t.element_size()
                                for t in {t.data_ptr(): t for t in bound.values()}.values())
        self.loaded = True

    # -------------------------------------------------------------------- cache
    def cache_requests(self) -> List[list]:
        """What each schedule entry asks of the cache."""
        return [self.layers[entry.layer].cache_requests() for entry in self.schedule]

    def cache_sources(self) -> List:
        return [entry.cache_from for entry in self.schedule]

    def launch_signature(self, rows: int, longest: int) -> tuple:
        """The launch choices of every layer for a decode step of `rows` sequences of at most
        `longest` tokens: a captured step may be replayed while this stays the same."""
        return tuple(layer.launch_signature(rows, longest) for layer in self.layers)

    # ------------------------------------------------------------------ forward
    def forward(self, ctx) -> torch.Tensor:
        """Runs the rows of `ctx` and returns float32 logits [wanted rows, vocab]."""
        stream = ResidualStream(self.embedding.forward(ctx.tables.tokens, ctx))
        for position in self.env.positions.values():
            position.on_embeddings(stream, ctx)
        for index, entry in enumerate(self.schedule):
            layer = self.layers[entry.layer]
            options = {}
            if getattr(layer, "supports_next_norm", False) and index + 1 < len(self.schedule):
                # The norm that reads the stream next: the layer's last product may prepare its rows.
                following = self.layers[self.schedule[index + 1].layer]
                options["next_norm"] = following.first_norm() if hasattr(following, "first_norm") else None
            layer.forward(stream, ctx, ctx.cache.views(index), entry.cache_from is None, **options)
        if ctx.plan.n_want == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.env.device)
        normed = self.final_norm.forward(stream, rows=ctx.tables.want_rows)
        return self.head.forward(normed, ctx)


def declared_parameters(spec: ModelSpec) -> List[Tuple[str, ParamSpec]]:
    """The tensors a model of this spec declares (no device memory is touched)."""
    return CausalLM(spec, torch.bfloat16, torch.device("cpu")).parameters()
