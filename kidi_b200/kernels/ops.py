"""Python faces of the CUDA kernels.

Each function checks shapes, element types and contiguity on the host, hands raw
device pointers and the current stream to the compiled launcher, and raises if the
launcher refuses the arguments or the launch fails. There is no CPU path: a tensor
that is not on a CUDA device is an error.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc.build import load_library
from ..errors import invalid_argument, runtime_error, unsupported

F32, BF16, NONE = 0, 1, -1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

c_void_p, c_int, c_float, c_longlong, c_ulonglong = (
    ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_ulonglong)


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise unsupported(f"the kernels take float32 and bfloat16, not {dtype}") from None


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(tensor: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(tensor.data_ptr() if tensor is not None else 0)


def _need_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for tensor in tensors:
        if tensor is not None and not tensor.is_cuda:
            raise runtime_error("the kernels run on a CUDA device only (there is no CPU path)")


launch_count = 0  # kernels of this package launched (or captured into a graph) so far
_launch_log: Optional[list] = None


class record_launches:
    """Collects, while it is open, the name of every kernel this package launches and of every
    product handed to the vendor library (`library_mm`), in order: `with record_launches() as
    names: ...`. Names carry the form a launcher chose, e.g. `attention_decode[ring]`, so that a
    test can assert which branch of a dispatch ran."""

    def __enter__(self) -> list:
        global _launch_log
        self._outer, _launch_log = _launch_log, []
        return _launch_log

    def __exit__(self, *exc) -> None:
        global _launch_log
        inner, _launch_log = _launch_log, self._outer
        if self._outer is not None:
            self._outer.extend(inner)


def note(what: str) -> None:
    """Records work that is not one of this package's kernels (a vendor-library product)."""
    if _launch_log is not None:
        _launch_log.append(what)


def _check(status: int, what: str, launches: int = 1) -> None:
    global launch_count
    if status == 0:
        launch_count += launches
        if _launch_log is not None:
            _launch_log.append(what)
        return
    if status == -2:
        raise unsupported(f"{what}: this combination of element types is not compiled")
    if status == -3:
        raise unsupported(f"{what}: a size lies outside what the kernel takes")
    if status < 0:
        raise unsupported(f"{what}: refused ({status})")
    raise runtime_error(f"{what}: CUDA error {status} at launch")


_core = None


def core():
    """The core kernel library, compiled at the first call."""
    global _core
    if _core is None:
        lib = load_library("core")
        lib.kidi_embedding.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p]
        lib.kidi_add_rmsnorm.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                         c_int, c_int, c_float, c_int, c_void_p]
        lib.kidi_silu_gate.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.kidi_gemm_simt.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                       c_longlong, c_longlong, c_longlong, c_void_p, c_void_p]
        lib.kidi_add_bias.argtypes = [c_void_p, c_int, c_void_p, c_int, c_int, c_longlong, c_void_p]
        lib.kidi_apply_row_factors.argtypes = [c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_float, c_void_p,
                                               c_int, c_int, c_void_p]
        lib.kidi_rope_store.argtypes = [c_void_p, c_int, c_int, c_void_p]
        lib.kidi_attention_generic.argtypes = [c_void_p, c_int, c_void_p]
        lib.kidi_argmax.argtypes = [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]
        lib.kidi_sample.argtypes = [c_void_p, c_void_p, c_int, c_int, c_void_p, c_ulonglong, c_void_p, c_void_p,
                                    c_void_p, c_void_p]
        lib.kidi_argmax_slices.argtypes = [c_int]
        lib.kidi_argmax_slices.restype = c_int
        lib.kidi_advance_decode.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                            c_void_p]
        for name in ("kidi_embedding", "kidi_add_rmsnorm", "kidi_silu_gate", "kidi_gemm_simt", "kidi_add_bias",
                     "kidi_apply_row_factors", "kidi_rope_store",
                     "kidi_attention_generic", "kidi_argmax", "kidi_sample", "kidi_advance_decode"):
            getattr(lib, name).restype = c_int
        _core = lib
    return _core


# ----------------------------------------------------------------- structures
class CacheGeometry(ctypes.Structure):
    _fields_ = [("table", c_void_p), ("pages_per_seq", c_int), ("page_shift", c_int), ("ring_pages", c_int),
                ("kv_heads", c_int), ("head_dim", c_int)]


class RopeStoreArgs(ctypes.Structure):
    _fields_ = [("qkv", c_void_p), ("ld", c_longlong), ("q_norm", c_void_p), ("k_norm", c_void_p),
                ("cos_table", c_void_p), ("sin_table", c_void_p), ("row_seq", c_void_p), ("row_pos", c_void_p),
                ("seq_slot", c_void_p), ("seq_start", c_void_p), ("seq_len", c_void_p), ("k_cache", c_void_p),
                ("v_cache", c_void_p), ("cache", CacheGeometry), ("rows", c_int), ("heads", c_int),
                ("kv_heads", c_int), ("head_dim", c_int), ("rotary_dim", c_int), ("eps", c_float), ("transform", c_int)]


class AttentionArgs(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("ldq", c_longlong), ("k_step", c_void_p), ("v_step", c_void_p),
                ("ldkv", c_longlong), ("k_cache", c_void_p), ("v_cache", c_void_p), ("cache", CacheGeometry),
                ("out", c_void_p), ("ldo", c_longlong), ("row_seq", c_void_p), ("row_pos", c_void_p),
                ("seq_slot", c_void_p), ("seq_start", c_void_p), ("seq_row0", c_void_p), ("rows", c_int),
                ("heads", c_int), ("kv_heads", c_int), ("head_dim", c_int), ("window", c_int), ("scale", c_float),
                ("softcap", c_float), ("slopes", c_void_p)]


def cache_geometry(view, kv_heads: int, head_dim: int) -> CacheGeometry:
    """The geometry of a `KVView` (or an empty one when there is no cache)."""
    if view is None:
        return CacheGeometry(0, 0, 0, 0, kv_heads, head_dim)
    page_size = view.page_size
    return CacheGeometry(view.table.data_ptr(), view.table.shape[1], page_size.bit_length() - 1, view.ring_pages,
                         kv_heads, head_dim)


# -------------------------------------------------------------------- kernels
def embedding(tokens: torch.Tensor, table: torch.Tensor, scale: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r, :] = table[tokens[r], :] * scale, in float32 (the residual stream)."""
    _need_cuda(tokens, table)
    if tokens.dtype != torch.int32 or tokens.dim() != 1 or not tokens.is_contiguous():
        raise invalid_argument("embedding takes a contiguous int32 vector of token ids")
    if table.dim() != 2 or not table.is_contiguous():
        raise invalid_argument("the embedding table must be a contiguous matrix")
    rows, (vocab, hidden) = tokens.shape[0], table.shape
    if out is None:
        out = torch.empty((rows, hidden), dtype=torch.float32, device=table.device)
    _check(core().kidi_embedding(_ptr(out), _ptr(table), dtype_code(table.dtype), _ptr(tokens), rows, hidden, vocab,
                                 float(scale), _stream()), "embedding")
    return out


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, row_index: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """residual += delta (in place, float32), then y = rmsnorm(residual) * weight.
    With `row_index`, row r of the output is computed from row row_index[r] and the
    residual is left as it is."""
    _need_cuda(residual, delta, weight, row_index)
    if residual.dtype != torch.float32 or residual.dim() != 2 or not residual.is_contiguous():
        raise invalid_argument("the residual stream is a contiguous float32 matrix")
    rows_in, hidden = residual.shape
    if delta is not None and (delta.shape != residual.shape or not delta.is_contiguous()):
        raise invalid_argument("the residual delta must match the residual stream")
    if weight.shape != (hidden,) or not weight.is_contiguous():
        raise invalid_argument(f"the norm weight must have {hidden} elements")
    if row_index is not None:
        if row_index.dtype != torch.int32 or row_index.dim() != 1:
            raise invalid_argument("row_index must be an int32 vector")
        rows = row_index.shape[0]
    else:
        rows = rows_in
    if out is None:
        out = torch.empty((rows, hidden), dtype=out_dtype, device=residual.device)
    _check(core().kidi_add_rmsnorm(
        _ptr(residual), _ptr(delta), dtype_code(delta.dtype) if delta is not None else NONE, _ptr(weight),
        dtype_code(weight.dtype), _ptr(out), dtype_code(out.dtype), _ptr(row_index), rows, hidden, float(eps),
        0 if row_index is not None else 1, _stream()), "add_rmsnorm")
    return out


def silu_gate(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:]."""
    _need_cuda(gate_up)
    if gate_up.dim() != 2 or gate_up.shape[1] % 2 or not gate_up.is_contiguous():
        raise invalid_argument("silu_gate takes a contiguous [rows, 2*I] matrix")
    rows, inter = gate_up.shape[0], gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    _check(core().kidi_silu_gate(_ptr(gate_up), _ptr(out), dtype_code(gate_up.dtype), rows, inter, _stream()),
           "silu_gate")
    return out


def check_bias(bias: Optional[torch.Tensor], features: int) -> None:
    if bias is not None and (bias.dtype != torch.float32 or bias.shape != (features,) or not bias.is_contiguous()):
        raise invalid_argument(f"a bias is a contiguous float32 vector of {features} elements")


def add_bias(y: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """y[r, :] += bias, in place (after a product the vendor library computed)."""
    _need_cuda(y, bias)
    if y.dim() != 2 or y.stride(1) != 1:
        raise invalid_argument("add_bias takes a matrix with contiguous rows")
    check_bias(bias, y.shape[1])
    _check(core().kidi_add_bias(_ptr(y), dtype_code(y.dtype), _ptr(bias), y.shape[0], y.shape[1], y.stride(0),
                                _stream()), "add_bias")
    return y


def apply_row_factors(values: torch.Tensor, parts: torch.Tensor, width: int, eps: float) -> torch.Tensor:
    """values[r, :] / sqrt(sum(parts[r, :]) / width + eps) as a new bfloat16 matrix: rows that were stored
    without their norm's factor, made plain."""
    _need_cuda(values, parts)
    if values.dtype != torch.bfloat16 or values.dim() != 2 or values.stride(1) != 1:
        raise invalid_argument("apply_row_factors takes a bfloat16 matrix with contiguous rows")
    if parts.dtype != torch.float32 or parts.dim() != 2 or parts.shape[0] != values.shape[0] or parts.stride(1) != 1:
        raise invalid_argument("apply_row_factors takes float32 parts, one row of them per row of values")
    out = torch.empty(values.shape, dtype=torch.bfloat16, device=values.device)
    _check(core().kidi_apply_row_factors(_ptr(values), values.stride(0), _ptr(parts), parts.shape[1], parts.stride(0),
                                         int(width), float(eps), _ptr(out), values.shape[0], values.shape[1],
                                         _stream()), "apply_row_factors")
    return out


def gemm_simt(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype,
              out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x @ weight.T (+ bias) with 32-bit fused multiply-adds in ascending k."""
    _need_cuda(x, weight, bias)
    check_bias(bias, weight.shape[0])
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1]:
        raise invalid_argument(f"gemm: x {tuple(x.shape)} does not fit weight {tuple(weight.shape)}")
    if x.stride(1) != 1 or weight.stride(1) != 1:
        raise invalid_argument("gemm: rows must be contiguous")
    M, K = x.shape
    N = weight.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    _check(core().kidi_gemm_simt(_ptr(x), dtype_code(x.dtype), _ptr(weight), dtype_code(weight.dtype), _ptr(out),
                                 dtype_code(out.dtype), M, N, K, x.stride(0), weight.stride(0), out.stride(0),
                                 _ptr(bias), _stream()), "gemm_simt")
    return out


def rope_store(qkv: torch.Tensor, *, heads: int, kv_heads: int, head_dim: int, q_norm: Optional[torch.Tensor],
               k_norm: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
               rotary_dim: int, tables, kv_view, store: bool, transform: bool = True) -> None:
    """In place on qkv [rows, (heads + 2*kv_heads) * head_dim]: per-head RMSNorm and
    rotation of the q and k heads; k and v heads are also written to the cache when
    `store` is set. With `transform=False` nothing is normalised or rotated: the k and v
    heads are only copied to the cache. `tables` is the step's `DeviceTables`."""
    _need_cuda(qkv)
    rows = qkv.shape[0]
    if qkv.dim() != 2 or qkv.stride(1) != 1 or qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
        raise invalid_argument("rope_store: qkv has the wrong shape")
    if (q_norm is None) != (k_norm is None):
        raise invalid_argument("rope_store: q_norm and k_norm come together")
    norm_dtype = q_norm.dtype if q_norm is not None else torch.float32
    if q_norm is not None and (q_norm.shape != (head_dim,) or k_norm.shape != (head_dim,) or k_norm.dtype != norm_dtype):
        raise invalid_argument("rope_store: the head norms must have head_dim elements and one type")
    if cos is not None and (cos.dtype != torch.float32 or cos.shape[1] != rotary_dim // 2 or sin.shape != cos.shape):
        raise invalid_argument("rope_store: the rotation tables must be float32 [positions, rotary_dim/2]")
    view = kv_view if store else None
    if view is not None and view.keys.dtype != qkv.dtype:
        raise invalid_argument("rope_store: the cache and the activations differ in element type")
    args = RopeStoreArgs(
        qkv.data_ptr(), qkv.stride(0), _ptr(q_norm), _ptr(k_norm), _ptr(cos), _ptr(sin),
        tables.row_seq.data_ptr(), tables.row_pos.data_ptr(), tables.seq_slot.data_ptr(),
        tables.seq_start.data_ptr(), tables.seq_len.data_ptr(),
        view.keys.data_ptr() if view is not None else 0, view.values.data_ptr() if view is not None else 0,
        cache_geometry(view, kv_heads, head_dim), rows, heads, kv_heads, head_dim, rotary_dim, float(eps),
        1 if transform else 0)
    _check(core().kidi_rope_store(ctypes.byref(args), dtype_code(qkv.dtype), dtype_code(norm_dtype), _stream()),
           "rope_store")


def attention_generic(qkv: torch.Tensor, out: torch.Tensor, *, heads: int, kv_heads: int, head_dim: int,
                      scale: float, window: Optional[int], tables, kv_view, keys_in_step: bool,
                      softcap: float = 0.0, slopes: Optional[torch.Tensor] = None) -> None:
    """Causal attention of every row of the step over its sequence's keys. Keys of the
    step's own rows are read from `qkv` when `keys_in_step` is set, earlier ones (or
    all of them) from the cache. `softcap` > 0 bounds a score s to softcap * tanh(s / softcap);
    `slopes` (float32 [heads]) adds slopes[h] * (key position - query position) to head h's scores."""
    if slopes is not None and (slopes.dtype != torch.float32 or slopes.shape != (heads,) or not slopes.is_contiguous()
                               or slopes.device != qkv.device):
        raise invalid_argument("attention: the score slopes must be a float32 vector with one entry per head")
    _need_cuda(qkv, out)
    rows = qkv.shape[0]
    if out.shape != (rows, heads * head_dim) or out.dtype != qkv.dtype or out.stride(1) != 1:
        raise invalid_argument("attention: the output has the wrong shape or type")
    if kv_view is None and not keys_in_step:
        raise invalid_argument("attention: there is neither a cache nor keys in the step")
    item = qkv.element_size()
    k_step = qkv.data_ptr() + heads * head_dim * item if keys_in_step else 0
    v_step = qkv.data_ptr() + (heads + kv_heads) * head_dim * item if keys_in_step else 0
    args = AttentionArgs(
        qkv.data_ptr(), qkv.stride(0), k_step, v_step, qkv.stride(0),
        kv_view.keys.data_ptr() if kv_view is not None else 0, kv_view.values.data_ptr() if kv_view is not None else 0,
        cache_geometry(kv_view, kv_heads, head_dim), out.data_ptr(), out.stride(0),
        tables.row_seq.data_ptr(), tables.row_pos.data_ptr(), tables.seq_slot.data_ptr(),
        tables.seq_start.data_ptr(), tables.seq_row0.data_ptr(), rows, heads, kv_heads, head_dim,
        int(window or 0), float(scale), float(softcap or 0.0), slopes.data_ptr() if slopes is not None else 0)
    _check(core().kidi_attention_generic(ctypes.byref(args), dtype_code(qkv.dtype), _stream()), "attention")


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need_cuda(logits)
    if logits.dtype != torch.float32 or logits.dim() != 2 or not logits.is_contiguous():
        raise invalid_argument("argmax takes a contiguous float32 [rows, vocab] matrix")
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    scratch, launches = _argmax_scratch(rows, vocab, logits.device)
    _check(core().kidi_argmax(_ptr(logits), _ptr(out), rows, vocab, _ptr(scratch), _stream()), "argmax", launches)
    return out


def _argmax_scratch(rows: int, vocab: int, device):
    """Scratch for the two-stage argmax of a wide vocabulary (None when one stage does)."""
    slices = core().kidi_argmax_slices(vocab)
    if slices == 1:
        return None, 1
    return torch.empty(2 * rows * slices, dtype=torch.float32, device=device), 2


def sample(logits: torch.Tensor, temperature: torch.Tensor, seed: int, keys: torch.Tensor, steps: torch.Tensor,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row: argmax where temperature is 0, else a draw from
    softmax(logits / temperature) keyed by (seed, keys[r], steps[r])."""
    _need_cuda(logits, temperature, keys, steps)
    if logits.dtype != torch.float32 or logits.dim() != 2 or not logits.is_contiguous():
        raise invalid_argument("sample takes a contiguous float32 [rows, vocab] matrix")
    rows, vocab = logits.shape
    if (temperature.dtype != torch.float32 or keys.dtype != torch.int64 or steps.dtype != torch.int32
            or temperature.shape != (rows,) or keys.shape != (rows,) or steps.shape != (rows,)):
        raise invalid_argument("sample: temperature float32, keys int64 and steps int32, one per row")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    scratch, launches = _argmax_scratch(rows, vocab, logits.device)
    _check(core().kidi_sample(_ptr(logits), _ptr(out), rows, vocab, _ptr(temperature),
                              ctypes.c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF), _ptr(keys), _ptr(steps), _ptr(scratch),
                              _stream()), "sample", launches + 1)
    return out


def advance_decode(tokens: torch.Tensor, selected: torch.Tensor, row_seq: torch.Tensor, row_pos: torch.Tensor,
                   seq_start: torch.Tensor, steps: torch.Tensor, vocab: int) -> None:
    """After a decode step: every live row takes its selected token as its next input
    and moves one position on (tokens, positions and step counters change in place)."""
    _need_cuda(tokens, selected, row_seq, row_pos, seq_start, steps)
    rows = tokens.shape[0]
    for tensor in (tokens, selected, row_seq, row_pos, seq_start, steps):
        if tensor.dtype != torch.int32 or tensor.shape[0] < rows:
            raise invalid_argument("advance_decode takes int32 vectors of one length")
    _check(core().kidi_advance_decode(_ptr(tokens), _ptr(selected), _ptr(row_seq), _ptr(row_pos), _ptr(seq_start),
                                      _ptr(steps), rows, vocab, _stream()), "advance_decode")
