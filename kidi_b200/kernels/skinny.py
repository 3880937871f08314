"""The weight-streaming bfloat16 matrix product for few rows (the decode step).

`fits` says whether a product can take this kernel: bfloat16 on both sides, at most
`MAX_ROWS` rows, 16-byte aligned rows. `MAX_ROWS` can be lowered or raised with the
environment variable KIDI_B200_SKINNY_MAX_ROWS (0 switches the kernel off).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from ..errors import invalid_argument
from . import ops
from .ops import _check, _need_cuda, _ptr, _stream, c_float, c_int, c_longlong, c_void_p, dtype_code

MAX_ROWS = int(os.environ.get("KIDI_B200_SKINNY_MAX_ROWS", "8"))
class Extras(ctypes.Structure):
    """KidiSkinnyExtras: the row factors of a product after a norm and the targets of a product
    before one (csrc/gemm_skinny.cu)."""
    _fields_ = [("factor_parts", c_void_p), ("factor_count", c_int), ("factor_stride", c_int),
                ("factor_width", c_int), ("factor_eps", c_float), ("residual", c_void_p), ("ld_residual", c_longlong),
                ("norm_weight", c_void_p), ("norm_weight_is_float", c_int), ("normed", c_void_p),
                ("ld_normed", c_longlong), ("parts_out", c_void_p), ("parts_stride", c_int)]


_bound = False


def _library():
    global _bound
    lib = ops.core()
    if not _bound:
        lib.kidi_gemm_skinny.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong,
                                         c_longlong, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p]
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
    return x.dim() == 2 and x.shape[0] <= MAX_ROWS and supports(x, weight)


def _row_tiles(features: int, rows: int, device) -> int:
    """The form of the kernel's blocks: 1: a tile of 16 weight rows and eight warps (two such
    blocks fit an SM); 4: the same tile and four warps (four fit), taken for up to 8 batch rows
    when the tiles are more than one round of the heavy blocks and at most one of the light
    ones, whose second, mostly empty round of heavy blocks would cost more than the light
    blocks' shallower prefetch."""
    from .attention import sm_count
    blocks = -(-features // 16)
    slots = 2 * sm_count(device)
    return 4 if rows <= 8 and slots < blocks <= 2 * slots else 1


def _factor_fields(extras: Extras, factors) -> None:
    """`factors`: (parts [rows, count] float32, width, eps) of rows that lack their norm's factor."""
    if factors is None:
        return
    parts, width, eps = factors
    if parts.dtype != torch.float32 or parts.dim() != 2 or parts.stride(1) != 1:
        raise invalid_argument("row factors come as float32 parts [rows, count]")
    extras.factor_parts, extras.factor_count, extras.factor_stride = parts.data_ptr(), parts.shape[1], parts.stride(0)
    extras.factor_width, extras.factor_eps = int(width), float(eps)


def gemm(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype, out: Optional[torch.Tensor] = None,
         row_tiles: Optional[int] = None, bias: Optional[torch.Tensor] = None, factors=None) -> torch.Tensor:
    """y = x @ weight.T (+ bias, float32) for x [M <= 64, K], weight [N, K], both bfloat16. With
    `factors` = (parts, width, eps) every row m of the result is multiplied by
    1 / sqrt(sum(parts[m]) / width + eps) first (the factor that an RMSNorm left out of x)."""
    _need_cuda(x, weight, bias)
    ops.check_bias(bias, weight.shape[0])
    if not supports(x, weight) or x.shape[1] != weight.shape[1]:
        raise invalid_argument("gemm_skinny: the operands do not fit this kernel")
    M, K = x.shape
    N = weight.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    extras = Extras()
    _factor_fields(extras, factors)
    _check(_library().kidi_gemm_skinny(_ptr(x), _ptr(weight), _ptr(out), dtype_code(out.dtype), M, N, K, x.stride(0),
                                       weight.stride(0), out.stride(0), 0, row_tiles or _row_tiles(N, M, x.device), _ptr(bias),
                                       ctypes.byref(extras), _stream()),
           "gemm_skinny[row factors]" if factors is not None else "gemm_skinny")
    return out


def gemm_into_residual(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor,
                       bias: Optional[torch.Tensor] = None, factors=None):
    """residual += x @ weight.T (+ bias) in place (float32 [M, N]); returns (normed, parts): normed
    [M, N] bfloat16 = the new residual times `norm_weight`, not yet normalised, and parts
    [M, ceil(N / 16)] float32, whose sum over a row is the sum of squares of the new residual's
    row. A product given `factors=(parts, N, eps)` normalises what it makes of `normed`."""
    _need_cuda(x, weight, residual, norm_weight, bias)
    ops.check_bias(bias, weight.shape[0])
    if not supports(x, weight) or x.shape[1] != weight.shape[1]:
        raise invalid_argument("gemm_into_residual: the operands do not fit this kernel")
    M, K = x.shape
    N = weight.shape[0]
    if residual.dtype != torch.float32 or residual.shape != (M, N) or residual.stride(1) != 1:
        raise invalid_argument("gemm_into_residual: the residual stream is float32 [rows, features]")
    if norm_weight.shape != (N,) or not norm_weight.is_contiguous() or norm_weight.dtype not in (torch.float32, torch.bfloat16):
        raise invalid_argument("gemm_into_residual: the norm weight has one float32 or bfloat16 element per feature")
    count = -(-N // 16)
    normed = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    parts = torch.empty((M, count), dtype=torch.float32, device=x.device)
    extras = Extras()
    _factor_fields(extras, factors)
    extras.residual, extras.ld_residual = residual.data_ptr(), residual.stride(0)
    extras.norm_weight, extras.norm_weight_is_float = norm_weight.data_ptr(), int(norm_weight.dtype == torch.float32)
    extras.normed, extras.ld_normed = normed.data_ptr(), normed.stride(0)
    extras.parts_out, extras.parts_stride = parts.data_ptr(), parts.stride(0)
    _check(_library().kidi_gemm_skinny(_ptr(x), _ptr(weight), None, dtype_code(torch.bfloat16), M, N, K, x.stride(0),
                                       weight.stride(0), 0, 0, _row_tiles(N, M, x.device), _ptr(bias),
                                       ctypes.byref(extras), _stream()),
           "gemm_skinny[into the residual]")
    return normed, parts


def gemm_silu_gate(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
                   row_tiles: int = 0, factors=None) -> torch.Tensor:
    """silu(x @ Wg.T) * (x @ Wu.T) for weight = [Wg; Wu] of shape [2I, K] (`factors`: as in `gemm`)."""
    _need_cuda(x, weight)
    if not supports(x, weight) or x.shape[1] != weight.shape[1] or weight.shape[0] % 2:
        raise invalid_argument("gemm_silu_gate: the operands do not fit this kernel")
    M, K = x.shape
    inter = weight.shape[0] // 2
    if out is None:
        out = torch.empty((M, inter), dtype=torch.bfloat16, device=x.device)
    extras = Extras()
    _factor_fields(extras, factors)
    _check(_library().kidi_gemm_skinny(_ptr(x), _ptr(weight), _ptr(out), dtype_code(out.dtype), M, inter, K,
                                       x.stride(0), weight.stride(0), out.stride(0), 1, row_tiles, None,
                                       ctypes.byref(extras), _stream()),
           "gemm_silu_gate[skinny]")
    return out
