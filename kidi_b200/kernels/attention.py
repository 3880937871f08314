"""Chooses and launches the attention kernel for a step.

The generic kernel takes every element type, head width up to 256 and any number of
heads, for prompts and for single tokens; it is the only one the 32-bit engine uses.
The bfloat16 engine uses the tensor-core kernels, which are compiled for the head
width of the loaded model at the first call: a prefill kernel for steps that bring
several tokens per sequence and a split-key decode kernel for steps of one token per
sequence. Setting KIDI_B200_GENERIC_ATTENTION=1 forces the generic kernel.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional

import torch

from ..csrc.build import load_library
from . import ops
from .ops import CacheGeometry, _check, c_float, c_int, c_longlong, c_void_p, cache_geometry

FORCE_GENERIC = os.environ.get("KIDI_B200_GENERIC_ATTENTION", "0") == "1"
# One token per sequence: the decode kernel normalises and rotates q and the new key itself and
# writes the new key and value to the cache (one kernel less per layer); 0 switches that off.
FUSE_ROTATION = os.environ.get("KIDI_B200_FUSE_ROTATION", "1") == "1"
# The page-copying decode kernel keeps a ring of three tiles (keys and values in turn), so that
# four blocks of head width 128 fit an SM (0: two key and two value tiles, three blocks).
# "force": wherever the kernel has that form (for tests of it on small batches).
DECODE_RING = os.environ.get("KIDI_B200_DECODE_RING", "1") in ("1", "force")
DECODE_RING_ALWAYS = os.environ.get("KIDI_B200_DECODE_RING", "1") == "force"
# Up to this many splits merge inside a thread-block cluster (no workspace, no second kernel);
# 0 switches that off.
CLUSTER_SPLITS = int(os.environ.get("KIDI_B200_CLUSTER_SPLITS", "8"))
TENSOR_MEMORY_PREFILL = os.environ.get("KIDI_B200_TCGEN05_ATTENTION", "1") == "1"
TENSOR_MEMORY_HEAD_DIMS = (64, 128)


class FastAttentionArgs(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("ldq", c_longlong), ("k_step", c_void_p), ("v_step", c_void_p),
                ("ldkv", c_longlong), ("k_cache", c_void_p), ("v_cache", c_void_p), ("cache", CacheGeometry),
                ("out", c_void_p), ("ldo", c_longlong), ("row_seq", c_void_p), ("row_pos", c_void_p),
                ("seq_slot", c_void_p), ("seq_start", c_void_p), ("seq_len", c_void_p), ("seq_row0", c_void_p),
                ("rows", c_int), ("seqs", c_int), ("heads", c_int), ("kv_heads", c_int), ("window", c_int),
                ("scale", c_float), ("partial_out", c_void_p), ("partial_stat", c_void_p), ("splits", c_int),
                ("counters", c_void_p), ("fuse", c_int), ("norm_is_float", c_int), ("q_norm", c_void_p),
                ("k_norm", c_void_p), ("cos_table", c_void_p), ("sin_table", c_void_p), ("rotary_dim", c_int),
                ("eps", c_float), ("cache_rows", c_longlong)]


_libraries: Dict[int, ctypes.CDLL] = {}
_tensor_memory_libraries: Dict[int, ctypes.CDLL] = {}
_sm_count: Dict[int, int] = {}
_ring_set: Dict[int, bool] = {}      # the decode form each library was last switched to


def library(head_dim: int) -> ctypes.CDLL:
    """The tensor-core attention kernels compiled for one head width."""
    lib = _libraries.get(head_dim)
    if lib is None:
        lib = load_library(f"attention_d{head_dim}", ("attention_bf16.cu",), {"KIDI_HEAD_DIM": head_dim})
        lib.kidi_attention_prefill.argtypes = [c_void_p, c_int, c_void_p]
        lib.kidi_attention_decode.argtypes = [c_void_p, c_void_p]
        lib.kidi_attention_prefill.restype = lib.kidi_attention_decode.restype = c_int
        lib.kidi_attention_decode_ring.argtypes = [c_int]
        lib.kidi_attention_decode_ring.restype = None
        lib.kidi_attention_decode_ring(0)
        _ring_set[head_dim] = False
        _libraries[head_dim] = lib
    return lib


def tensor_memory_library(head_dim: int) -> ctypes.CDLL:
    """The tcgen05 prompt-attention kernel compiled for one head width (64 or 128)."""
    lib = _tensor_memory_libraries.get(head_dim)
    if lib is None:
        lib = load_library(f"attention_tcgen05_d{head_dim}", ("attention_tcgen05.cu",), {"KIDI_HEAD_DIM": head_dim})
        lib.kidi_attention_prefill_tcgen05.argtypes = [
            c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
            c_float, c_void_p, c_void_p]
        lib.kidi_attention_prefill_tcgen05.restype = c_int
        lib.kidi_attention_tcgen05_timeout_flag.restype = c_int
        _tensor_memory_libraries[head_dim] = lib
    return lib


def tensor_memory_fits(qkv: torch.Tensor, out: torch.Tensor, head_dim: int, heads: int, kv_heads: int,
                       scale: float = 1.0) -> bool:
    """Prompts whose keys are all rows of the step, in bfloat16 with 16-byte aligned rows."""
    return (TENSOR_MEMORY_PREFILL and scale > 0 and not FORCE_GENERIC and head_dim in TENSOR_MEMORY_HEAD_DIMS
            and qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and heads % kv_heads == 0
            and qkv.stride(1) == 1 and out.stride(1) == 1 and qkv.stride(0) % 8 == 0 and out.stride(0) % 8 == 0
            and qkv.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)


class PromptCache(ctypes.Structure):
    """Where the keys and values lie when prompts continue cached sequences (KidiPromptCache)."""
    _fields_ = [("keys", c_void_p), ("values", c_void_p), ("rows", c_longlong), ("table", c_void_p),
                ("pages_per_seq", c_int), ("seq_start", c_void_p), ("seq_slot", c_void_p)]


def prefill_tensor_memory(qkv: torch.Tensor, out: torch.Tensor, seq_len: torch.Tensor, seq_row0: torch.Tensor,
                          seqs: int, max_new: int, *, heads: int, kv_heads: int, head_dim: int, scale: float,
                          window: int, kv_view=None, seq_start: Optional[torch.Tensor] = None,
                          seq_slot: Optional[torch.Tensor] = None) -> None:
    """Causal attention of packed prompts. Without `kv_view` the prompts start at position 0
    and every key is a row of qkv; with it (a cache of 64-token pages without a ring, into
    which the step's rows have been written) every key and value is read from the cache,
    so the prompts may continue sequences of `seq_start` tokens."""
    lib = tensor_memory_library(head_dim)
    cache = None
    if kv_view is not None:
        cache = PromptCache(kv_view.keys.data_ptr(), kv_view.values.data_ptr(), kv_view.keys.numel() // head_dim,
                            kv_view.table.data_ptr(), kv_view.table.shape[1], seq_start.data_ptr(), seq_slot.data_ptr())
    _check(lib.kidi_attention_prefill_tcgen05(
        qkv.data_ptr(), qkv.stride(0), qkv.shape[0], out.data_ptr(), out.stride(0), seq_len.data_ptr(),
        seq_row0.data_ptr(), seqs, max_new, heads, kv_heads, int(window or 0), float(scale),
        ctypes.byref(cache) if cache is not None else None, ops._stream()),
        "attention_prefill_tcgen05")


def timeout_flags() -> int:
    """Non-zero when a bounded wait in one of the loaded attention libraries ran out."""
    found = 0
    for lib in _libraries.values():
        lib.kidi_attention_timeout_flag.restype = c_int
        found |= int(lib.kidi_attention_timeout_flag() != 0)
    for lib in _tensor_memory_libraries.values():
        found |= int(lib.kidi_attention_tcgen05_timeout_flag() != 0)
    return found


def fast_fits(dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int, decode: bool) -> bool:
    if FORCE_GENERIC or dtype != torch.bfloat16 or head_dim % 16 or head_dim > 256 or heads % kv_heads:
        return False
    return not decode or heads // kv_heads <= 16


def sm_count(device: torch.device) -> int:
    index = device.index if device.index is not None else \
        (torch.cuda.current_device() if torch.cuda.is_available() else 0)
    if index not in _sm_count:
        _sm_count[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_count[index]


def ring_available(head_dim: int) -> bool:
    return DECODE_RING and head_dim % 64 == 0


def blocks_per_sm(head_dim: int = 128, ring: bool = False) -> int:
    """Decode attention blocks that fit one SM: 8 query rows, the tiles (four 64-row tiles with
    rows padded by 8 elements, or with `ring` three unpadded ones), what a cluster's blocks send
    each other and a kilobyte of the system's; at most four by registers. Three at head width
    128, four with the ring."""
    received = (8 * head_dim + 32 + 128) * 4 + 128
    if ring:
        block = 1024 + (3 * 64 * head_dim + 8 * (head_dim + 8)) * 2 + received + 1024
    else:
        block = (8 + 4 * 64) * (head_dim + 8) * 2 + received + 1024
    return max(1, min(4, (228 * 1024) // block))


def decode_ring(rows: int, kv_heads: int, device: torch.device, head_dim: int) -> bool:
    """Whether decode attention takes its ring form: one block per (row, key/value head), no
    splits. The ring holds fewer bytes in flight per block and pays a second barrier per
    tile, so it is taken only where one more block per SM saves a round of blocks."""
    if not ring_available(head_dim):
        return False
    if DECODE_RING_ALWAYS:
        return True
    items, sms = max(1, rows * kv_heads), sm_count(device)
    with_ring, without = blocks_per_sm(head_dim, True) * sms, blocks_per_sm(head_dim, False) * sms
    return -(-items // with_ring) < -(-items // without)


# What a block spends beside its tiles (launch, tables, query, merge of the splits), in tile
# times, fitted to kernel times measured on a B200 (batch 1 to 64, 300 to 16,000 tokens): less
# when the splits merge inside a thread-block cluster than through a workspace.
FIXED_COST_TILES = 14.0
FIXED_COST_TILES_CLUSTER = 3.5


def decode_splits(rows: int, kv_heads: int, longest: int, device: torch.device, head_dim: int = 128) -> int:
    """How many blocks share a sequence's keys. A block walks its 64-key pages one after
    another, so the kernel's time is (waves of blocks) x (pages per block + a fixed cost);
    the number of splits that makes this smallest is chosen, at most one per page."""
    pages = max(1, -(-longest // 64))
    forced = int(os.environ.get("KIDI_B200_DECODE_SPLITS", "0"))
    if forced:
        return max(1, min(pages, forced))
    if decode_ring(rows, kv_heads, device, head_dim):
        return 1
    slots = blocks_per_sm(head_dim) * sm_count(device)
    items = max(1, rows * kv_heads)
    best, best_cost = 1, None
    for splits in range(1, min(pages, 32) + 1):
        clustered = 1 < splits <= CLUSTER_SPLITS and items * splits <= slots
        fixed = FIXED_COST_TILES_CLUSTER if clustered else FIXED_COST_TILES
        cost = -(-items * splits // slots) * (-(-pages // splits) + fixed)
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = splits, cost
    return best


def fuses_rotation(plan, qkv: torch.Tensor, *, heads: int, kv_heads: int, head_dim: int, kv_view, q_norm, k_norm,
                   cos, sin, rotary_dim: int) -> bool:
    """Whether `run` can take the step's rows as the projection left them (`rotation=`):
    one token per sequence over a paged bfloat16 cache, at most eight query heads per
    key/value head, and norm weights and angle tables that 16-byte vectors can read."""
    if not (FUSE_ROTATION and plan.is_decode and kv_view is not None and kv_view.page_size == 64
            and fast_fits(qkv.dtype, heads, kv_heads, head_dim, True) and heads // kv_heads <= 8):
        return False
    if (q_norm is None) != (k_norm is None) or qkv.stride(0) % 8 or qkv.data_ptr() % 16:
        return False
    if q_norm is not None and (q_norm.dtype != k_norm.dtype or q_norm.dtype not in (torch.float32, torch.bfloat16)
                               or not q_norm.is_contiguous() or not k_norm.is_contiguous()):
        return False
    if cos is not None and (rotary_dim % 16 or rotary_dim > head_dim or cos.dtype != torch.float32
                            or cos.data_ptr() % 16 or sin.data_ptr() % 16 or not cos.is_contiguous()):
        return False
    return True


def run(ctx, qkv, out, *, heads, kv_heads, head_dim, scale, window, kv_view, keys_in_step, rotation=None,
        step_rows_cached: bool = False, splits: Optional[int] = None, ring: Optional[bool] = None,
        softcap: float = 0.0, slopes: Optional[torch.Tensor] = None) -> None:
    """`ctx` gives the step's `plan`, its device `tables` and `workspace(name, count, zero)`.
    `keys_in_step`: the step's own keys and values are read from qkv (else from the
    cache, like the earlier ones). `step_rows_cached`: they are in the cache as well (a cache
    that keeps every page is written before attention), so a kernel may read everything
    from there. `rotation` (only where `fuses_rotation` said yes): dict(q_norm, k_norm, eps,
    cos, sin, rotary_dim, store): the kernel normalises and rotates q and the step's key
    and, with `store`, writes the step's key and value to the cache. `splits` and `ring`
    override the launcher's own choice of the decode kernel's form (tests of each form)."""
    plan, tables = ctx.plan, ctx.tables
    decode = plan.is_decode and not keys_in_step
    # Scores that are bounded or shifted by position run on the general kernel (the tensor-core kernels
    # compute plain scaled scores).
    reshaped = bool(softcap) or slopes is not None
    if (reshaped or not fast_fits(qkv.dtype, heads, kv_heads, head_dim, decode)
            or (kv_view is not None and kv_view.page_size != 64)):
        ops.attention_generic(qkv, out, heads=heads, kv_heads=kv_heads, head_dim=head_dim, scale=scale,
                              window=window, tables=tables, kv_view=kv_view, keys_in_step=keys_in_step,
                              softcap=softcap, slopes=slopes)
        return
    if not decode and tensor_memory_fits(qkv, out, head_dim, heads, kv_heads, scale):
        common = dict(heads=heads, kv_heads=kv_heads, head_dim=head_dim, scale=scale, window=window)
        if keys_in_step and int(plan.seq_start.max()) == 0:      # every key is a row of this step
            prefill_tensor_memory(qkv, out, tables.seq_len, tables.seq_row0, plan.n_seqs, plan.max_new, **common)
            return
        # Prompts that continue cached sequences: the step's rows are in the cache already (a
        # cache that keeps every page is written before attention), so every key comes from there.
        if (kv_view is not None and (step_rows_cached or not keys_in_step) and kv_view.ring_pages == 0
                and kv_view.page_size == 64 and kv_view.keys.is_contiguous() and kv_view.table.is_contiguous()):
            prefill_tensor_memory(qkv, out, tables.seq_len, tables.seq_row0, plan.n_seqs, plan.max_new, kv_view=kv_view,
                                  seq_start=tables.seq_start, seq_slot=tables.seq_slot, **common)
            return
    item = qkv.element_size()
    args = FastAttentionArgs(
        qkv.data_ptr(), qkv.stride(0),
        qkv.data_ptr() + heads * head_dim * item if keys_in_step else 0,
        qkv.data_ptr() + (heads + kv_heads) * head_dim * item if keys_in_step else 0, qkv.stride(0),
        kv_view.keys.data_ptr() if kv_view is not None else 0, kv_view.values.data_ptr() if kv_view is not None else 0,
        cache_geometry(kv_view, kv_heads, head_dim), out.data_ptr(), out.stride(0),
        tables.row_seq.data_ptr(), tables.row_pos.data_ptr(), tables.seq_slot.data_ptr(), tables.seq_start.data_ptr(),
        tables.seq_len.data_ptr(), tables.seq_row0.data_ptr(), qkv.shape[0], plan.n_seqs, heads, kv_heads,
        int(window or 0), float(scale), 0, 0, 1, 0)
    lib = library(head_dim)
    stream = ops._stream()
    if not decode:
        _check(lib.kidi_attention_prefill(ctypes.byref(args), plan.max_new, stream), "attention_prefill[mma.sync]")
        return
    rows = qkv.shape[0]
    splits, ring = decode_form(rows, kv_heads, head_dim, plan.max_total, window, qkv.device, splits, ring)
    if _ring_set.get(head_dim) != ring:                # the form is a switch of the library, not of a launch
        lib.kidi_attention_decode_ring(1 if ring else 0)
        _ring_set[head_dim] = ring
    # One wave of blocks and few splits: the blocks of a (row, key/value head) form a thread-block
    # cluster and merge through distributed shared memory. Clusters that must wait for several
    # free slots of one GPC at once lose that again when the grid takes more than a wave.
    one_wave = rows * kv_heads * splits <= blocks_per_sm(head_dim, ring) * sm_count(qkv.device)
    clustered = 1 < splits <= CLUSTER_SPLITS and heads // kv_heads <= 8 and one_wave
    form = "ring" if ring else "one block" if splits == 1 else "cluster" if clustered else "combine kernel"
    if splits > 1 and not clustered:
        workspace = ctx.workspace("attention_partial", rows * heads * splits * (head_dim + 2))
        args.partial_out = workspace.data_ptr()
        args.partial_stat = workspace.data_ptr() + rows * heads * splits * head_dim * 4
        # One wave of blocks: the last block of each (row, key/value head) merges its splits at
        # the kernel's tail. More waves: a second kernel merges (the fence and the counter would
        # hold up every block's slot).
        if heads // kv_heads <= 8 and splits <= 32 and one_wave:
            # Zeroed when it is made; the kernel leaves every counter at zero.
            args.counters = ctx.workspace("attention_counters", rows * kv_heads, zero=True).data_ptr()
            form = "merge in the last block"
    args.splits = splits
    args.cache_rows = kv_view.keys.numel() // head_dim if kv_view.keys.is_contiguous() else 0
    if rotation is not None:
        args.k_step = qkv.data_ptr() + heads * head_dim * item
        args.v_step = qkv.data_ptr() + (heads + kv_heads) * head_dim * item
        args.fuse = 1 | (2 if rotation.get("store", True) else 0)
        q_norm, k_norm, cos, sin = (rotation.get(name) for name in ("q_norm", "k_norm", "cos", "sin"))
        if q_norm is not None:
            args.q_norm, args.k_norm = q_norm.data_ptr(), k_norm.data_ptr()
            args.norm_is_float = int(q_norm.dtype == torch.float32)
        if cos is not None:
            args.cos_table, args.sin_table = cos.data_ptr(), sin.data_ptr()
            args.rotary_dim = int(rotation["rotary_dim"])
        args.eps = float(rotation.get("eps", 0.0))
    _check(lib.kidi_attention_decode(ctypes.byref(args), stream), f"attention_decode[{form}]",
           2 if form == "combine kernel" else 1)


def decode_form(rows: int, kv_heads: int, head_dim: int, longest: int, window, device: torch.device,
                splits: Optional[int] = None, ring: Optional[bool] = None):
    """(key splits, ring form) of decode attention for `rows` sequences of at most `longest`
    tokens; `splits` / `ring`, when given, replace the policy's choice."""
    reach = min(longest, int(window)) + 64 if window else longest
    if splits is None:
        splits = decode_splits(rows, kv_heads, reach, device, head_dim)
    if ring is None:
        ring = splits == 1 and decode_ring(rows, kv_heads, device, head_dim)
    return splits, bool(ring) and ring_available(head_dim)


class AttentionLauncher:
    """What an attention part owns of the kernels: its geometry, the choice of kernel for a step
    and the launch. Each part (hence each group of layers with a geometry of its own) chooses the
    form of its decode kernel itself, from the rows of the step and the longest sequence."""

    def __init__(self, *, heads: int, kv_heads: int, head_dim: int, scale: float, window=None,
                 softcap: float = 0.0, slopes: Optional[torch.Tensor] = None):
        self.geometry = dict(heads=heads, kv_heads=kv_heads, head_dim=head_dim)
        self.scale, self.window = scale, window
        # Scores bounded by softcap * tanh(s / softcap), or shifted by slopes[head] * (key - query position):
        # such scores run on the general kernel.
        self.softcap, self.slopes = float(softcap or 0.0), slopes
        self.reshaped = bool(self.softcap) or slopes is not None

    def fuses_rotation(self, plan, qkv, **arguments) -> bool:
        """Whether `run` can do norm, rotation and the cache write of this step itself."""
        return not self.reshaped and fuses_rotation(plan, qkv, **self.geometry, **arguments)

    def run(self, ctx, qkv, out, **arguments) -> None:
        run(ctx, qkv, out, scale=self.scale, window=self.window, softcap=self.softcap, slopes=self.slopes,
            **self.geometry, **arguments)

    def launch_signature(self, dtype: torch.dtype, rows: int, longest: int, device: torch.device) -> tuple:
        """What a captured decode step freezes of this launcher's choices: the form of the
        tensor-core decode kernel (the general kernel, which the 32-bit engine runs, has none)."""
        geometry = self.geometry
        if self.reshaped or not fast_fits(dtype, geometry["heads"], geometry["kv_heads"], geometry["head_dim"], True):
            return ()
        return decode_form(rows, geometry["kv_heads"], geometry["head_dim"], longest, self.window, device)
