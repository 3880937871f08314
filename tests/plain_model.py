"""A plain, slow implementation of dense Qwen3, written from the reference's formulas.

It rests on the formulas only: the reference's own model code cannot be imported or
compiled here (its tensor maths lives in a third-party submodule that is not part of
the tree, and its Qwen3 is a bidirectional INT8 backbone without cache or head), so
there is no run of it to compare with. Every function cites the file and line of the
formula it restates.

Whole sequences, no cache, one function per part, float32 (or float64) on the CPU with
elementary tensor operations. It shares no code with `kidi_b200`: it reads config.json
keys and checkpoint tensors by itself.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


# --------------------------------------------------------------------- loading
def read_model_folder(model_dir: str):
    """config.json as a dict and the tensors of model.safetensors by name
    (folder contract: src/kidi/checkpoint/config.cpp:234-256)."""
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as handle:
        config = json.load(handle)
    return config, load_file(os.path.join(model_dir, "model.safetensors"))


# ----------------------------------------------------------------------- parts
def embed(tokens: Sequence[int], table: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    """h0[t] = E[token[t]] * 1.0  (src/kidi/model/qwen3.cpp:78,134-136;
    src/kidi/layers/gemma4.cpp:97-99,132-142)."""
    return table.to(dtype)[torch.as_tensor(list(tokens), dtype=torch.long)] * 1.0


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * (1/sqrt(sum(x^2)/H + eps)) * w over the last axis
    (src/kidi/runtime/mps/eager_kernels.metal:65-87; src/kidi/layers/gemma4.cpp:23-67)."""
    width = x.shape[-1]
    inverse = 1.0 / torch.sqrt((x * x).sum(dim=-1, keepdim=True) / width + eps)
    return x * inverse * weight.to(x.dtype)


def rotary_tables(length: int, head_dim: int, theta: float):
    """freq_i = 1/theta^(2i/d); angle = float(position) * freq_i; cos, sin; all in
    32-bit (src/kidi/model/qwen3.cpp:146-157)."""
    half = head_dim // 2
    frequency = np.empty(half, dtype=np.float32)
    for i in range(half):
        # powf of the C library: the correctly rounded 32-bit power of the 32-bit base and exponent.
        power = np.float32(np.power(np.float64(np.float32(theta)), np.float64(np.float32(2 * i) / np.float32(head_dim))))
        frequency[i] = np.float32(1.0) / power
    angle = np.arange(length, dtype=np.float32)[:, None] * frequency[None, :]
    return torch.from_numpy(np.cos(angle).astype(np.float32)), torch.from_numpy(np.sin(angle).astype(np.float32))


def norm_then_rotate(x: torch.Tensor, weight: torch.Tensor, eps: float, cos: torch.Tensor,
                     sin: torch.Tensor) -> torch.Tensor:
    """Per head: RMSNorm over head_dim, then out_c = n_c cos_j + r_c sin_j with
    j = c mod half, r_c = -n_{c+half} (c < half) or n_{c-half}
    (src/kidi/layers/qwen3.cpp:37-48; src/kidi/ops/context.cpp:1051-1065;
    src/kidi/runtime/mps/eager_kernels.metal:87-97). x: [T, heads, d]; cos, sin: [T, d/2]."""
    normed = rms_norm(x, weight, eps)
    half = x.shape[-1] // 2
    rotated = torch.cat([-normed[..., half:], normed[..., :half]], dim=-1)
    cos_full = torch.cat([cos, cos], dim=-1).to(x.dtype)[:, None, :]
    sin_full = torch.cat([sin, sin], dim=-1).to(x.dtype)[:, None, :]
    return normed * cos_full + rotated * sin_full


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int] = None) -> torch.Tensor:
    """s[t,u] = (q[t,h] . k[u,h // group]) / sqrt(d) + mask; softmax over u; sum p v
    (src/kidi/layers/qwen3.cpp:53-54; src/kidi/runtime/vulkan/attention.comp:32-101).
    The mask is the generic causal one, 0 where u <= t and -1e9 elsewhere
    (src/kidi/model/gemma4.cpp:736-740); with a window W also -1e9 where u <= t - W.
    q: [T, heads, d], k, v: [T, kv_heads, d] -> [T, heads * d]."""
    length, heads, width = q.shape
    group = heads // k.shape[1]
    scale = 1.0 / math.sqrt(float(width))
    t = torch.arange(length)[:, None]
    u = torch.arange(length)[None, :]
    visible = u <= t
    if window is not None:
        visible = visible & (u > t - window)
    mask = torch.where(visible, 0.0, -1e9).to(q.dtype)
    out = torch.empty(length, heads, width, dtype=q.dtype)
    for head in range(heads):
        scores = (q[:, head, :] @ k[:, head // group, :].T) * scale + mask
        top = scores.max(dim=-1, keepdim=True).values
        weights = torch.exp(scores - top)
        weights = weights / weights.sum(dim=-1, keepdim=True)
        out[:, head, :] = weights @ v[:, head // group, :]
    return out.reshape(length, heads * width)


def attention_layer(x: torch.Tensor, tensors: Dict[str, torch.Tensor], prefix: str, config: dict, cos, sin,
                    window: Optional[int]) -> torch.Tensor:
    """q, k, v projections without bias, per-head norm + rotation of q and k (not v),
    attention, output projection (src/kidi/layers/qwen3.cpp:32-56)."""
    heads, kv_heads, width = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
    eps = config["rms_norm_eps"]
    length = x.shape[0]
    w = lambda name: tensors[prefix + name].to(x.dtype)
    q = (x @ w("q_proj.weight").T).reshape(length, heads, width)
    k = (x @ w("k_proj.weight").T).reshape(length, kv_heads, width)
    v = (x @ w("v_proj.weight").T).reshape(length, kv_heads, width)
    q = norm_then_rotate(q, w("q_norm.weight"), eps, cos, sin)
    k = norm_then_rotate(k, w("k_norm.weight"), eps, cos, sin)
    return causal_attention(q, k, v, window) @ w("o_proj.weight").T


def gated_feed_forward(x: torch.Tensor, tensors: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """f = (g / (1 + exp(-g))) * u with g = x Wg^T, u = x Wu^T; y = f Wd^T
    (src/kidi/layers/gemma4.cpp:206-224; src/kidi/runtime/mps/eager_kernels.metal:129-137)."""
    w = lambda name: tensors[prefix + name].to(x.dtype)
    gate = x @ w("gate_proj.weight").T
    up = x @ w("up_proj.weight").T
    return (gate / (1.0 + torch.exp(-gate)) * up) @ w("down_proj.weight").T


def block(x: torch.Tensor, tensors, layer: int, config: dict, cos, sin, window) -> torch.Tensor:
    """h = x + attention(input_norm(x)); out = h + mlp(post_attention_norm(h))
    (src/kidi/layers/qwen3.cpp:111-122)."""
    prefix = f"model.layers.{layer}."
    eps = config["rms_norm_eps"]
    hidden = x + attention_layer(rms_norm(x, tensors[prefix + "input_layernorm.weight"], eps), tensors,
                                 prefix + "self_attn.", config, cos, sin, window)
    return hidden + gated_feed_forward(rms_norm(hidden, tensors[prefix + "post_attention_layernorm.weight"], eps),
                                       tensors, prefix + "mlp.")


def layer_window(config: dict, layer: int) -> Optional[int]:
    kinds = config.get("layer_types")
    if kinds and kinds[layer] == "sliding_attention":
        return int(config["sliding_window"])
    return None


def rope_theta(config: dict) -> float:
    parameters = config.get("rope_parameters")
    return float(parameters["rope_theta"] if parameters else config["rope_theta"])


def forward(config: dict, tensors: Dict[str, torch.Tensor], tokens: Sequence[int], dtype=torch.float32,
            schedule: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence: embeddings, every block, final norm
    (src/kidi/model/qwen3.cpp:181-204), then the head, logits = norm(h) Wlm^T with Wlm the
    embedding table when tie_word_embeddings is set (ours; precedent
    src/kidi/model/gemma4.cpp:769-778). `schedule` lists the layers in run order
    (default: each layer once, in order)."""
    cos, sin = rotary_tables(len(tokens), config["head_dim"], rope_theta(config))
    hidden = embed(tokens, tensors["model.embed_tokens.weight"], dtype)
    order = list(schedule) if schedule is not None else list(range(config["num_hidden_layers"]))
    for layer in order:
        hidden = block(hidden, tensors, layer, config, cos, sin, layer_window(config, layer))
    hidden = rms_norm(hidden, tensors["model.norm.weight"], config["rms_norm_eps"])
    head = tensors["model.embed_tokens.weight"] if config.get("tie_word_embeddings", False) else tensors["lm_head.weight"]
    return hidden @ head.to(dtype).T


# -------------------------------------------------------------------- sampling
def greedy_token(logits: Sequence[float]) -> int:
    """Largest value, ties to the lowest index; NaN, +inf or no finite value: -1
    (ARCHITECTURE.md:612-616; src/kidi/inference/decoder.cpp:72-80)."""
    values = np.asarray(logits, dtype=np.float32)
    if np.isnan(values).any() or (values == np.inf).any() or not np.isfinite(values.max()):
        return -1
    return int(np.argmax(values))


def uniform_number(seed: int, key: int, step: int) -> float:
    """The uniform number in [0, 1) that the library draws for (seed, key, step): a
    splitmix64-style mix, top 24 bits (ours; the reference samples text greedily only)."""
    mask = (1 << 64) - 1
    z = (seed * 0x9E3779B97F4A7C15 + key * 0xBF58476D1CE4E5B9 + step * 0x94D049BB133111EB + 0x2545F4914F6CDD1D) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z = z ^ (z >> 31)
    return (z >> 40) / 16777216.0


def temperature_token(logits: Sequence[float], temperature: float, seed: int, key: int, step: int) -> int:
    """p = softmax(logits / T); the first index whose cumulative probability exceeds u."""
    if temperature <= 0:
        return greedy_token(logits)
    values = np.asarray(logits, dtype=np.float64)
    weights = np.exp((values - values.max()) / temperature)
    cumulative = np.cumsum(weights)
    target = uniform_number(seed, key, step) * cumulative[-1]
    return int(min(np.searchsorted(cumulative, target, side="right"), len(values) - 1))


def generate(config, tensors, prompt: Sequence[int], max_new_tokens: int, stop_ids: Sequence[int] = (),
             temperature: float = 0.0, seed: int = 0, key: int = 0, dtype=torch.float32) -> List[int]:
    """Token by token from whole-sequence forwards (no cache): the reference's greedy
    bookkeeping (src/kidi/inference/decoder.cpp:65-101): a stop token ends the
    sequence and is not appended; otherwise stop after max_new_tokens."""
    tokens = list(prompt)
    produced: List[int] = []
    for step in range(max_new_tokens):
        logits = forward(config, tensors, tokens, dtype)[-1].float().numpy()
        token = temperature_token(logits, temperature, seed, key, step)
        if token in stop_ids:
            break
        produced.append(token)
        tokens.append(token)
    return produced
