"""Ways of cutting the same requests into steps, and the comparison with the plain model."""
from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np
import torch

import plain_model
from kidi_b200 import StepBatch


def random_requests(vocab: int, lengths: Sequence[int], seed: int) -> Dict[str, List[int]]:
    generator = np.random.default_rng(seed)
    return {f"r{index}": generator.integers(0, vocab, size=length).tolist() for index, length in enumerate(lengths)}


def plain_logits(folder: str, requests: Dict[str, List[int]], dtype=torch.float32) -> Dict[str, np.ndarray]:
    config, tensors = plain_model.read_model_folder(folder)
    return {name: plain_model.forward(config, tensors, tokens, dtype).float().numpy()
            for name, tokens in requests.items()}


def run_whole(engine, requests) -> Dict[str, np.ndarray]:
    """Each request alone, its whole sequence in one step, logits everywhere."""
    out = {}
    for name, tokens in requests.items():
        slot = engine.acquire()
        logits = engine.step(StepBatch([slot], [tokens], [list(range(len(tokens)))]))
        out[name] = logits.cpu().numpy()
        engine.release(slot)
    return out


def run_chunked(engine, requests, chunk: int, batch_size: int = 2) -> Dict[str, np.ndarray]:
    """Batches of requests whose prompts come in chunks of `chunk` tokens: every step but the
    first continues sequences that the cache already holds, with several tokens each (a
    request that has run out brings nothing more and leaves the steps)."""
    out = {}
    names = list(requests)
    for begin in range(0, len(names), batch_size):
        batch = names[begin:begin + batch_size]
        slots = {name: engine.acquire() for name in batch}
        rows = {name: [] for name in batch}
        done = {name: 0 for name in batch}
        while any(done[name] < len(requests[name]) for name in batch):
            live = [name for name in batch if done[name] < len(requests[name])]
            pieces = [requests[name][done[name]:done[name] + chunk] for name in live]
            logits = engine.step(StepBatch([slots[name] for name in live], pieces,
                                           [list(range(len(piece))) for piece in pieces])).cpu().numpy()
            cursor = 0
            for name, piece in zip(live, pieces):
                rows[name].append(logits[cursor:cursor + len(piece)])
                cursor += len(piece)
                done[name] += len(piece)
        for name in batch:
            out[name] = np.concatenate(rows[name], axis=0)
            engine.release(slots[name])
    return out


def run_tail_decoded(engine, requests, tail: int = 32) -> Dict[str, np.ndarray]:
    """Each request alone: all but the last `tail` tokens in one step, the rest one by one."""
    out = {}
    for name, tokens in requests.items():
        slot = engine.acquire()
        head = max(1, len(tokens) - tail)
        rows = [engine.step(StepBatch([slot], [tokens[:head]], [list(range(head))])).cpu().numpy()]
        for position in range(head, len(tokens)):
            rows.append(engine.step(StepBatch([slot], [[tokens[position]]], [[0]])).cpu().numpy())
        out[name] = np.concatenate(rows, axis=0)
        engine.release(slot)
    return out


def run_batches(engine, requests, batch_size: int, prompt_fraction: float = 0.5) -> Dict[str, np.ndarray]:
    """Batches of unequal lengths, one after another so that slots are used again. A
    batch's requests start together with unequal prompts, then go on by one token a
    step; the shorter ones end earlier and give their slots back at once."""
    names = list(requests)
    out: Dict[str, List[np.ndarray]] = {name: [] for name in names}
    for begin in range(0, len(names), batch_size):
        group = names[begin:begin + batch_size]
        slots = {name: engine.acquire() for name in group}
        heads = {name: max(1, int(len(requests[name]) * prompt_fraction)) for name in group}
        logits = engine.step(StepBatch([slots[n] for n in group], [requests[n][:heads[n]] for n in group],
                                       [list(range(heads[n])) for n in group])).cpu().numpy()
        cursor = 0
        for name in group:
            out[name].append(logits[cursor:cursor + heads[name]])
            cursor += heads[name]
        done = dict(heads)
        live = [name for name in group if done[name] < len(requests[name])]
        for name in group:
            if name not in live:
                engine.release(slots[name])
        while live:
            logits = engine.step(StepBatch([slots[n] for n in live], [[requests[n][done[n]]] for n in live],
                                           [[0] for _ in live])).cpu().numpy()
            for index, name in enumerate(live):
                out[name].append(logits[index:index + 1])
                done[name] += 1
            for name in [n for n in live if done[n] >= len(requests[n])]:
                engine.release(slots[name])
            live = [name for name in live if done[name] < len(requests[name])]
    return {name: np.concatenate(parts, axis=0) for name, parts in out.items()}


def relative_error(found: np.ndarray, expected: np.ndarray) -> float:
    """Largest absolute difference over the larger of 1 and the largest expected magnitude."""
    return float(np.abs(found - expected).max() / max(1.0, float(np.abs(expected).max())))


def first_bad_position(found: np.ndarray, expected: np.ndarray, tolerance: float):
    scale = max(1.0, float(np.abs(expected).max()))
    errors = np.abs(found - expected).max(axis=1) / scale
    bad = np.nonzero(errors > tolerance)[0]
    return (int(bad[0]), float(errors[bad[0]])) if bad.size else None


def rms_error(found: Dict[str, np.ndarray], expected: Dict[str, np.ndarray]) -> float:
    """Root of the mean squared difference over every logit of every request, each request's
    differences relative to the larger of 1 and its largest expected magnitude."""
    total, count = 0.0, 0
    for name, reference in expected.items():
        scale = max(1.0, float(np.abs(reference).max()))
        total += float((((found[name] - reference) / scale) ** 2).sum())
        count += reference.size
    return (total / max(count, 1)) ** 0.5


def worst_error(found: Dict[str, np.ndarray], expected: Dict[str, np.ndarray]) -> float:
    return max(relative_error(found[name], reference) for name, reference in expected.items())


def assert_matches(found: Dict[str, np.ndarray], expected: Dict[str, np.ndarray], tolerance, what: str):
    """`tolerance`: the largest relative difference allowed, or a pair of that and a bound on the
    root mean square of all differences (a fault that moves many logits a little shows there)."""
    rms_bound = None
    if isinstance(tolerance, tuple):
        tolerance, rms_bound = tolerance
    for name, reference in expected.items():
        assert found[name].shape == reference.shape, f"{what}: {name} has shape {found[name].shape}"
        assert np.isfinite(found[name]).all(), f"{what}: {name} holds a non-finite logit"
        bad = first_bad_position(found[name], reference, tolerance)
        assert bad is None, (f"{what}: request {name} (length {reference.shape[0]}) first differs at position "
                             f"{bad[0]} with relative error {bad[1]:.3e} > {tolerance:.1e}")
    if rms_bound is not None:
        rms = rms_error(found, expected)
        assert rms <= rms_bound, f"{what}: root mean square error {rms:.3e} > {rms_bound:.1e}"
