"""The weight-streaming bfloat16 matrix product for few rows (the decode step).

`fits` says whether a product can take this kernel: bfloat16 on both sides, at most
`MAX_ROWS` rows, 16-byte aligned rows. `MAX_ROWS` can be lowered or raised with the
environment variable KIDI_B200_SKINNY_MAX_ROWS (0 switches the kernel off).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..errors import invalid_argument
from . import ops
from .ops import _check, _need_cuda, _ptr, _stream, c_int, c_longlong, c_void_p, dtype_code

MAX_ROWS = int(os.environ.get("KIDI_B200_SKINNY_MAX_ROWS", "8"))
LIBRARY_BAND = tuple(int(v) for v in os.environ.get("KIDI_B200_SKINNY_LIBRARY_BAND", "296,768").split(","))

_bound = False


def _library():
    global _bound
    lib = ops.core()
    if not _bound:
        lib.kidi_gemm_skinny.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong,
                                         c_longlong, c_longlong, c_int, c_int, c_void_p, c_void_p]
        lib.kidi_gemm_skinny.restype = c_int
        _bound = True
    return lib


def supports(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the kernel can take the product at all (up to 64 rows)."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2 and weight.dim() == 2
            and 0 < x.shape[0] <= 64 and x.shape[1] % 8 == 0 and x.stride(1) == 1 and weight.stride(1) == 1
            and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and weight.data_ptr() % 16 == 0)


def fits(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the product should take this kernel: it can, and it has few enough rows
    for streaming the weights once to beat the matrix library."""
    if not (x.dim() == 2 and x.shape[0] <= MAX_ROWS and supports(x, weight)):
        return False
    # Between one and three and a half waves of blocks (a tile of 16 weight rows per block, two
    # blocks per SM) the last, partly filled wave costs more than the vendor library loses
    # elsewhere: measured on a B200 at 6144 x 4096, 14.7 against 12.0 microseconds.
    blocks = -(-weight.shape[0] // 16)
    return not (LIBRARY_BAND[0] < blocks < LIBRARY_BAND[1])


def _row_tiles(features: int) -> int:
    # One tile of 16 weight rows per block: measured on a B200 it streams every shape of the
    # benchmark's model faster than two tiles do (the output head: 177 against 248 microseconds).
    return 1


def gemm(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype, out: Optional[torch.Tensor] = None,
         row_tiles: Optional[int] = None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x @ weight.T (+ bias, float32) for x [M <= 64, K], weight [N, K], both bfloat16."""
    _need_cuda(x, weight, bias)
    ops.check_bias(bias, weight.shape[0])
    if not supports(x, weight) or x.shape[1] != weight.shape[1]:
        raise invalid_argument("gemm_skinny: the operands do not fit this kernel")
    M, K = x.shape
    N = weight.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    _check(_library().kidi_gemm_skinny(_ptr(x), _ptr(weight), _ptr(out), dtype_code(out.dtype), M, N, K, x.stride(0),
                                       weight.stride(0), out.stride(0), 0, row_tiles or _row_tiles(N), _ptr(bias),
                                       _stream()),
           "gemm_skinny")
    return out


def gemm_silu_gate(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
                   row_tiles: int = 0) -> torch.Tensor:
    """silu(x @ Wg.T) * (x @ Wu.T) for weight = [Wg; Wu] of shape [2I, K]."""
    _need_cuda(x, weight)
    if not supports(x, weight) or x.shape[1] != weight.shape[1] or weight.shape[0] % 2:
        raise invalid_argument("gemm_silu_gate: the operands do not fit this kernel")
    M, K = x.shape
    inter = weight.shape[0] // 2
    if out is None:
        out = torch.empty((M, inter), dtype=torch.bfloat16, device=x.device)
    _check(_library().kidi_gemm_skinny(_ptr(x), _ptr(weight), _ptr(out), dtype_code(out.dtype), M, inter, K,
                                       x.stride(0), weight.stride(0), out.stride(0), 1, row_tiles, None, _stream()),
           "gemm_silu_gate[skinny]")
    return out
