"""The engine: a loaded model, its cache, and the one step function.

`Engine.step(batch)` is everything between a request's tokens and its next token's
logits. It runs only the tokens it is given, as one packed batch, against what
earlier steps left in the cache, and returns the logits at the wanted places. It is
the reference's generic causal contract folded into one call: `prefill`, `forward`
and `forward_batch_tokens` of src/kidi/model/model.h:106-150, with the step of
src/kidi/model/gemma4.cpp:981-1069 as the model for its order (validate, embed, per
layer write the cache and attend, head at the wanted rows, advance the positions
only when everything succeeded).
"""
from __future__ import annotations

from typing import Any, Dict, Mapping, Optional, Sequence

import torch

from ..cache.sequence_cache import SequenceCache
from ..config.reader import read_config_json
from ..errors import invalid_argument, runtime_error
from ..kernels import attention as attention_kernels
from ..registry import spec_from_config
from ..weights.loader import Checkpoint, TensorDict, bind_parameters
from ..weights.random_init import random_parameters
from .model import CausalLM
from .plan import StepBatch, StepPlan, build_plan

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
          torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


class DeviceTables:
    """The integer tables of a `StepPlan` on the device, as views of one buffer."""

    def __init__(self, buffer: torch.Tensor, offsets: Mapping[str, tuple]):
        for name, (begin, size) in offsets.items():
            setattr(self, name, buffer[begin:begin + size])


class StepContext:
    """What parts see of a step: the host tables (`plan`), the device tables (`tables`), the
    cache, the engine's element type and device, and scratch memory. It knows no kind of part."""

    def __init__(self, plan: StepPlan, tables: DeviceTables, cache: SequenceCache, dtype: torch.dtype,
                 device: torch.device, workspaces: Optional[Dict[str, torch.Tensor]] = None):
        self.plan, self.tables, self.cache, self.dtype, self.device = plan, tables, cache, dtype, device
        self._workspaces = workspaces if workspaces is not None else {}

    def workspace(self, name: str, count: int, zero: bool = False) -> torch.Tensor:
        """Scratch memory of at least `count` 32-bit elements that kernels of one step may
        use one after another (it is kept between steps and grows on demand). With `zero`
        it is filled with zeros when it is made; its users leave it zero."""
        held = self._workspaces.get(name)
        if held is None or held.numel() < count:
            make = torch.zeros if zero else torch.empty
            held = make(max(count, 1), dtype=torch.float32, device=self.device)
            self._workspaces[name] = held
        return held


class Engine:
    def __init__(self, model: CausalLM, *, max_tokens: int, max_slots: Optional[int] = None, config: Any = None):
        if not torch.cuda.is_available() or model.env.device.type != "cuda":
            raise runtime_error("this engine runs on a CUDA device (sm_100a); none is available")
        if not model.loaded:
            raise invalid_argument("the model has no weights yet")
        self.model = model
        self.config = config
        self.spec = model.spec
        self.dtype, self.device = model.env.dtype, model.env.device
        self.vocab_size = model.spec.vocab_size
        self.cache = SequenceCache(model.cache_requests(), max_tokens=max_tokens,
                                   max_positions=model.spec.max_positions, dtype=self.dtype, device=self.device,
                                   max_slots=max_slots, cache_from=model.cache_sources())
        self._staging = [None, None]      # pinned host buffers, used in turn
        self._staging_done = [None, None]  # events: the copy out of the buffer has finished
        self._turn = 0
        self._workspaces: Dict[str, torch.Tensor] = {}
        self._backends: Dict[tuple, object] = {}

    # ---------------------------------------------------------------- loading
    @classmethod
    def load(cls, model_dir: str, *, dtype="bfloat16", device="cuda:0", max_tokens: int = 4096,
             max_slots: Optional[int] = None, cast_weights: bool = False) -> "Engine":
        """From a folder with config.json and model.safetensors (or the shards its index
        names); config.json chooses the model. A tensor keeps the width the file stores it
        in; with `cast_weights` a bfloat16 engine rounds wider matrices to bfloat16."""
        engine_dtype = _dtype(dtype)
        _require_cuda(device)
        _, typed, spec = spec_from_config(read_config_json(model_dir))
        model = CausalLM(spec, engine_dtype, torch.device(device))
        checkpoint = Checkpoint(model_dir)
        try:
            with torch.cuda.device(model.env.device):
                model.bind(bind_parameters(model.parameters(), checkpoint, engine_dtype=engine_dtype,
                                           device=model.env.device, ignored=model.ignored_tensors(),
                                           cast_matrices=cast_weights))
        finally:
            checkpoint.close()
        return cls(model, max_tokens=max_tokens, max_slots=max_slots, config=typed)

    @classmethod
    def from_config(cls, config: Mapping[str, Any], *, seed: int = 0, dtype="bfloat16", device="cuda:0",
                    max_tokens: int = 4096, max_slots: Optional[int] = None,
                    tensors: Optional[Mapping[str, torch.Tensor]] = None, cast_weights: bool = False) -> "Engine":
        """From a config.json dictionary, with random weights drawn on the device from
        `seed`, or with the checkpoint tensors given in `tensors`."""
        engine_dtype = _dtype(dtype)
        _require_cuda(device)
        _, typed, spec = spec_from_config(config)
        model = CausalLM(spec, engine_dtype, torch.device(device))
        with torch.cuda.device(model.env.device):
            if tensors is not None:
                bound = bind_parameters(model.parameters(), TensorDict(tensors), engine_dtype=engine_dtype,
                                        device=model.env.device, ignored=model.ignored_tensors(),
                                        cast_matrices=cast_weights)
            else:
                bound = random_parameters(model.parameters(), seed, engine_dtype, model.env.device)
            model.bind(bound)
        return cls(model, max_tokens=max_tokens, max_slots=max_slots, config=typed)

    # ------------------------------------------------------------------ slots
    def acquire(self) -> int:
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    # ------------------------------------------------------------------- step
    def _upload(self, plan: StepPlan) -> DeviceTables:
        packed = plan.packed()
        turn = self._turn
        self._turn ^= 1
        if self._staging_done[turn] is not None:
            self._staging_done[turn].synchronize()
        staging = self._staging[turn]
        if staging is None or staging.numel() < packed.size:
            staging = torch.empty(max(1024, 2 * packed.size), dtype=torch.int32).pin_memory()
            self._staging[turn] = staging
        staging[:packed.size].copy_(torch.from_numpy(packed))
        buffer = torch.empty(packed.size, dtype=torch.int32, device=self.device)
        buffer.copy_(staging[:packed.size], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self._staging_done[turn] = event
        return DeviceTables(buffer, plan.offsets())

    def step(self, batch: StepBatch) -> torch.Tensor:
        """Runs one step and returns float32 logits [wanted places, vocab] on the
        device, in the order of the batch's sequences and of their `want` lists."""
        with torch.cuda.device(self.device):
            starts = [self.cache.length(slot) for slot in batch.slots]
            plan = build_plan(batch, starts, self.vocab_size)
            growth = [(slot, start + int(count)) for slot, start, count in zip(batch.slots, starts, plan.seq_len)]
            self.cache.reserve(growth)
            self.cache.flush_tables()
            ctx = StepContext(plan, self._upload(plan), self.cache, self.dtype, self.device, self._workspaces)
            logits = self.model.forward(ctx)
            self.cache.commit(growth)
            return logits

    # --------------------------------------------------------------- generation
    def generate(self, prompts: Sequence[Sequence[int]], *, max_new_tokens: int = 0, temperature: float = 0.0,
                 seed: int = 0, ignore_eos: bool = False, stop_ids: Sequence[int] = (), max_active: int = 0,
                 context_size: int = 0, prefill_chunk_size: int = 0, use_graph: bool = True,
                 max_tokens: Optional[Sequence[Optional[int]]] = None, stats=None, detailed: bool = False):
        """Generates for every prompt (lists of token ids, host integers) and returns the
        new token ids of each, in order; with `detailed`, `Generation` records instead.
        The model's own end tokens stop a sequence unless `ignore_eos` is set. `max_active`
        bounds the sequences of a batch (0: as many as the cache has slots and tokens for)."""
        from ..sampling.sampler import Sampler
        from .generate import EngineBackend, GenerationOptions, generate
        with torch.cuda.device(self.device):
            options = GenerationOptions(
                max_new_tokens=max_new_tokens, context_size=context_size, prefill_chunk_size=prefill_chunk_size,
                temperature=temperature, seed=seed, ignore_eos=ignore_eos, stop_ids=tuple(stop_ids),
                max_active=max_active or self.cache.n_slots, use_graph=use_graph)
            key = (seed, use_graph)
            backend = self._backends.get(key)
            if backend is None:
                backend = self._backends[key] = EngineBackend(self, Sampler(seed), use_graph)
            found = generate(backend, prompts, options, stop_ids=self.spec.eos_token_ids, max_tokens=max_tokens,
                             stats=stats)
            self.check_device_errors()
        return found if detailed else [generation.token_ids for generation in found]

    def check_device_errors(self) -> None:
        """Raises if a kernel gave up a bounded wait (its result would be wrong). Kernels
        that wait on barriers record that instead of hanging; this reads the records."""
        from ..kernels import tcgen05
        code = tcgen05.error_code(self.device)
        if code or attention_kernels.timeout_flags():
            raise runtime_error(f"a kernel gave up waiting for its data (matrix product code {code}); "
                                f"the results of this engine cannot be trusted")

    # ------------------------------------------------------------- accounting
    def memory(self) -> Dict[str, int]:
        return {"weight_bytes": self.model.weight_bytes, "cache_bytes": self.cache.bytes()}


def _require_cuda(device) -> None:
    if torch.device(device).type != "cuda" or not torch.cuda.is_available():
        raise runtime_error(f"this engine runs on a CUDA device (sm_100a) and has no CPU path; "
                            f"device '{device}' cannot be used here")


def _dtype(name) -> torch.dtype:
    try:
        return DTYPES[name]
    except KeyError:
        raise invalid_argument(f"dtype must be bfloat16 or float32, not {name!r}") from None
