"""The bfloat16 matrix product on the 5th-generation tensor cores (tcgen05, TMEM, TMA).

`gemm` / `gemm_silu_gate` compute y = x @ weight.T (or its fused SiLU gate) with the
weight as the instruction's M operand, so that any number of rows of x, from one decoded
token to a whole prompt, runs through the same kernel. With few rows the product is
bound by reading the weight once; the kernel then splits K over several blocks, which
needs a workspace and counters that this module keeps per device (allocated once, never
replaced, so that captured graphs can hold their addresses).

KIDI_B200_TCGEN05_MAX_ROWS bounds the rows for which `fits` says yes (0 switches the
kernel off); above it the caller uses the matrix library, which streams weights faster
from 17 rows on.
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

from ..errors import invalid_argument, runtime_error
from . import attention as attention_kernels
from . import ops
from .ops import _check, _need_cuda, _ptr, _stream, c_int, c_longlong, c_void_p, dtype_code

MAX_ROWS = int(os.environ.get("KIDI_B200_TCGEN05_MAX_ROWS", "16"))
MIN_FEATURES = 16384                    # the dispatcher uses this kernel for weights at least this tall
MIN_GATED_ROWS = 9                      # and its fused SiLU gate from this many rows on (below: the skinny kernel)
# The most rows for the fused gate (and within MAX_ROWS): beyond, the product followed by the gate kernel is faster.
MAX_GATED_ROWS = int(os.environ.get("KIDI_B200_TCGEN05_MAX_GATED_ROWS", "32"))
WORKSPACE_FLOATS = 8 * 1024 * 1024      # 32 MiB of partial tiles
COUNTERS = 16384

_bound = False
_state: Dict[int, tuple] = {}


def _library():
    global _bound
    lib = ops.core()
    if not _bound:
        lib.kidi_gemm_tcgen05.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong,
                                          c_longlong, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_void_p]
        lib.kidi_gemm_tcgen05.restype = c_int
        lib.kidi_gemm_tcgen05_token_tile.argtypes = [c_int]
        lib.kidi_gemm_tcgen05_token_tile.restype = c_int
        _bound = True
    return lib


def _device_state(device: torch.device):
    index = device.index if device.index is not None else torch.cuda.current_device()
    state = _state.get(index)
    if state is None:
        state = (torch.empty(WORKSPACE_FLOATS, dtype=torch.float32, device=device),
                 torch.zeros(COUNTERS, dtype=torch.int32, device=device),
                 torch.zeros(1, dtype=torch.int32, device=device))
        _state[index] = state
    return state


def error_code(device: torch.device) -> int:
    """The code a kernel left when one of its bounded waits ran out (0: none). Reading
    it synchronises with the device."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    state = _state.get(index)
    return int(state[2].item()) if state is not None else 0


def supports(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2 and weight.dim() == 2
            and x.shape[0] > 0 and x.shape[1] % 8 == 0 and x.stride(1) == 1 and weight.stride(1) == 1
            and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and weight.data_ptr() % 16 == 0)


def fits(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return x.dim() == 2 and x.shape[0] <= MAX_ROWS and supports(x, weight)


def choose_splits(rows: int, features: int, K: int, gated: bool, device: torch.device) -> int:
    """Blocks per tile: enough that about two blocks per SM stream weights, each with at
    least two 64-wide k-blocks, within the workspace."""
    lib = _library()
    tile = lib.kidi_gemm_tcgen05_token_tile(rows)
    span = 64 if gated else 128
    tiles = -(-features // span) * -(-rows // tile)
    k_blocks = -(-K // 64)
    wanted = (2 * attention_kernels.sm_count(device)) // max(1, tiles)
    splits = max(1, min(wanted, k_blocks // 2, 32))
    while splits > 1 and (tiles * splits * 128 * tile > WORKSPACE_FLOATS or tiles > COUNTERS):
        splits -= 1
    return splits


def _run(x, weight, out, features: int, gated: bool, splits: Optional[int], bias=None) -> None:
    _need_cuda(x, weight, out, bias)
    ops.check_bias(bias, features)
    rows, K = x.shape
    if splits is None:
        splits = choose_splits(rows, features, K, gated, x.device)
    workspace, counters, error = _device_state(x.device)
    _check(_library().kidi_gemm_tcgen05(
        _ptr(x), _ptr(weight), _ptr(out), dtype_code(out.dtype), rows, features, K, x.stride(0), weight.stride(0),
        out.stride(0), 1 if gated else 0, splits, _ptr(workspace), _ptr(counters), _ptr(error), _ptr(bias),
        _stream()),
        "gemm_silu_gate[tcgen05]" if gated else "gemm_tcgen05")


def gemm(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype, out: Optional[torch.Tensor] = None,
         splits: Optional[int] = None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x @ weight.T (+ bias, float32) for bfloat16 x [rows, K] and weight [features, K]; y bfloat16 or
    float32."""
    if not supports(x, weight) or x.shape[1] != weight.shape[1]:
        raise invalid_argument("gemm_tcgen05: the operands do not fit this kernel")
    if out is None:
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=x.device)
    _run(x, weight, out, weight.shape[0], False, splits, bias)
    return out


def gemm_silu_gate(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
                   splits: Optional[int] = None) -> torch.Tensor:
    """silu(x @ Wg.T) * (x @ Wu.T) for weight = [Wg; Wu] of shape [2I, K]."""
    if not supports(x, weight) or x.shape[1] != weight.shape[1] or weight.shape[0] % 2:
        raise invalid_argument("gemm_silu_gate (tcgen05): the operands do not fit this kernel")
    inter = weight.shape[0] // 2
    if out is None:
        out = torch.empty((x.shape[0], inter), dtype=torch.bfloat16, device=x.device)
    _run(x, weight, out, inter, True, splits)
    return out
