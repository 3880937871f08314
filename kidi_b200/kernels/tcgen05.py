"""The bfloat16 matrix product on the 5th-generation tensor cores (tcgen05, TMEM, TMA).

`gemm` / `gemm_silu_gate` compute y = x @ weight.T (or its fused SiLU gate) with the
weight as the instruction's M operand, so that any number of rows of x, from one decoded
token to a whole prompt, runs through the same kernel: persistent blocks, the accumulator
double-buffered in tensor memory, results written by TMA stores. With few rows the
product is bound by reading the weight once; the kernel then deals the k-blocks of the
tiles out over all blocks, which needs a workspace and counters that this module keeps
per device (allocated once, never replaced, so that captured graphs can hold their
addresses). Products of one device therefore must not overlap in time: the package issues
all its work on one stream; a caller with streams of its own orders the calls.

KIDI_B200_TCGEN05_MAX_ROWS bounds the rows for which `fits` says yes (0 switches the
kernel off); above it the caller uses the matrix library, which streams weights faster
from 17 rows on, except weights as tall as an output head (KIDI_B200_TCGEN05_MAX_ROWS_TALL).
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
# From this many rows on (prompts) every product runs here again: whole tiles of 128 features x 256
# tokens, one persistent block per SM (0 switches that off: the matrix library).
PROMPT_ROWS = int(os.environ.get("KIDI_B200_TCGEN05_PROMPT_ROWS", "1024"))
MIN_FEATURES = 16384                    # the dispatcher uses this kernel for weights at least this tall
# A weight as tall as an output head (over a thousand tiles: rounds of whole tiles, no shared ones) streams
# as fast as through the matrix library up to this many rows (151,936 x 4,096: 207 against 214 us at 24 and
# 32 rows, 214 against 213 at 64, with 32-bit results against the library's 16-bit ones).
TALL_FEATURES = 65536
MAX_ROWS_TALL = int(os.environ.get("KIDI_B200_TCGEN05_MAX_ROWS_TALL", "64"))
MIN_GATED_ROWS = 9                      # and its fused SiLU gate from this many rows on (below: the skinny kernel)
# The most rows for the fused gate (and within MAX_ROWS): beyond, the product followed by the gate kernel is faster.
MAX_GATED_ROWS = int(os.environ.get("KIDI_B200_TCGEN05_MAX_GATED_ROWS", "32"))
COUNTERS = 4096                         # two per block of a launch (two blocks an SM at most)

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
        lib.kidi_gemm_tcgen05_workspace.argtypes = [c_int, c_int, c_int, c_int, c_int]
        lib.kidi_gemm_tcgen05_workspace.restype = c_longlong
        _bound = True
    return lib


def _device_state(device: torch.device):
    """(workspace, counters, error word) of a device: allocated once and never replaced, so that
    captured graphs can hold their addresses. The workspace holds two partial tiles of 128
    features x 256 tokens for each of the blocks that are resident at once."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    state = _state.get(index)
    if state is None:
        floats = 2 * 2 * attention_kernels.sm_count(device) * 128 * 256
        state = (torch.empty(floats, dtype=torch.float32, device=device),
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
    if x.dim() != 2 or not supports(x, weight):
        return False
    return x.shape[0] <= MAX_ROWS or (x.shape[0] <= MAX_ROWS_TALL and weight.shape[0] >= TALL_FEATURES)


def fits_prompt(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Many rows (a prompt): the compute-bound form of the kernel."""
    return x.dim() == 2 and 0 < PROMPT_ROWS <= x.shape[0] and supports(x, weight)


def _run(x, weight, out, features: int, gated: bool, splits: Optional[int], bias=None) -> None:
    _need_cuda(x, weight, out, bias)
    ops.check_bias(bias, features)
    rows, K = x.shape
    splits = int(splits or 0)            # 0: as many blocks as the GPU holds at once
    workspace, counters, error = _device_state(x.device)
    if _library().kidi_gemm_tcgen05_workspace(rows, features, K, 1 if gated else 0, splits) > workspace.numel():
        raise runtime_error("gemm_tcgen05: the workspace of this device is too small for the launch")
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
