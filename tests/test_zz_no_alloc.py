"""The decode-attention entry point that allocates nothing, called through its exported
C symbol and compared with the ordinary entry point (whose workspace the caller
allocates). Two calls in a row, of different sizes, share the library's fixed workspace:
the second must not be disturbed by what the first left there. This file is collected
last, so that a run that stops at the first failure has run every other test before."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"


def make_case(rows, heads, kv_heads, head_dim, lengths, seed):
    """A filled cache, a query row per sequence and the argument block for decode attention."""
    from kidi_b200.cache.sequence_cache import KVRequest, SequenceCache
    from kidi_b200.engine.plan import StepBatch, build_plan
    from kidi_b200.kernels.attention import FastAttentionArgs
    from kidi_b200.kernels.ops import cache_geometry

    generator = torch.Generator().manual_seed(seed)
    cache = SequenceCache([[KVRequest(kv_heads, head_dim)]], max_tokens=8192, max_positions=2048,
                          dtype=torch.bfloat16, device=torch.device(DEVICE))
    slots = [cache.acquire() for _ in range(rows)]
    cache.reserve([(slot, length) for slot, length in zip(slots, lengths)])
    cache.flush_tables()
    view = cache.views(0)[0]
    view.keys.copy_(torch.randn(view.keys.shape, generator=generator).to(torch.bfloat16))
    view.values.copy_(torch.randn(view.values.shape, generator=generator).to(torch.bfloat16))
    plan = build_plan(StepBatch(slots, [[0]] * rows), [length - 1 for length in lengths], vocab_size=2)
    tables = {name: torch.from_numpy(getattr(plan, name)).to(DEVICE) for name in plan.FIELDS}
    width = (heads + 2 * kv_heads) * head_dim
    qkv = torch.randn(rows, width, generator=generator).to(torch.bfloat16).to(DEVICE)

    def arguments(out, splits, workspace, whole_pages=False):
        """`whole_pages`: the cache is told to be contiguous (cache_rows), so that the kernel takes
        its pages by TMA tensor copies instead of row by row."""
        count = rows * heads * splits
        block = FastAttentionArgs(
            qkv.data_ptr(), qkv.stride(0), 0, 0, qkv.stride(0), view.keys.data_ptr(), view.values.data_ptr(),
            cache_geometry(view, kv_heads, head_dim), out.data_ptr(), out.stride(0),
            tables["row_seq"].data_ptr(), tables["row_pos"].data_ptr(), tables["seq_slot"].data_ptr(),
            tables["seq_start"].data_ptr(), tables["seq_len"].data_ptr(), tables["seq_row0"].data_ptr(),
            rows, rows, heads, kv_heads, 0, 1.0 / math.sqrt(head_dim),
            workspace.data_ptr() if workspace is not None else 0,
            workspace.data_ptr() + count * head_dim * 4 if workspace is not None else 0, splits, 0)
        if whole_pages:
            block.cache_rows = view.keys.numel() // head_dim
        return block

    return arguments, (cache, tables, qkv)


def test_static_workspace_matches_the_allocating_entry_point():
    from kidi_b200.kernels import attention

    head_dim = 128
    lib = attention.library(head_dim)
    lib.kidi_attention_decode_static.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.kidi_attention_decode_static.restype = ctypes.c_int
    lib.kidi_attention_decode_static_need.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int]
    lib.kidi_attention_decode_static_need.restype = ctypes.c_longlong
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    cases = [dict(rows=6, heads=16, kv_heads=4, lengths=[1000, 64, 65, 333, 1, 700], splits=7, seed=1),
             dict(rows=3, heads=8, kv_heads=8, lengths=[129, 900, 400], splits=3, seed=2)]
    # Each case twice: pages copied row by row, then whole pages by TMA (both forms of the kernel
    # merge their splits through the fixed workspace).
    for case, whole_pages in [(case, form) for case in cases for form in (False, True)]:
        rows, heads, splits = case["rows"], case["heads"], case["splits"]
        arguments, keep = make_case(rows, heads, case["kv_heads"], head_dim, case["lengths"], case["seed"])
        need = lib.kidi_attention_decode_static_need(rows, heads, splits)
        assert need == rows * heads * splits * (head_dim + 2)
        expected = torch.zeros(rows, heads * head_dim, dtype=torch.bfloat16, device=DEVICE)
        workspace = torch.empty(need, dtype=torch.float32, device=DEVICE)
        block = arguments(expected, splits, workspace, whole_pages)
        assert lib.kidi_attention_decode(ctypes.byref(block), stream) == 0
        found = torch.zeros_like(expected)
        block = arguments(found, splits, None, whole_pages)        # no workspace from the caller
        assert lib.kidi_attention_decode_static(ctypes.byref(block), stream) == 0
        torch.cuda.synchronize()
        assert torch.isfinite(found.float()).all()
        error = float((found.float() - expected.float()).abs().max()) / max(1.0, float(expected.float().abs().max()))
        assert error <= 1e-2, error                                # the tolerance of the bfloat16 attention tests
        assert torch.equal(found, expected)                        # in fact the same kernels: the same bits

    # A request beyond the fixed workspace is refused and launches nothing.
    arguments, keep = make_case(2, 8, 8, head_dim, [100, 200], 3)
    out = torch.zeros(2, 8 * head_dim, dtype=torch.bfloat16, device=DEVICE)
    block = arguments(out, 1, None)
    block.rows, block.splits = 60000, 64                           # 60000 * 8 * 64 * 130 floats: far too many
    assert lib.kidi_attention_decode_static(ctypes.byref(block), stream) == -3
    # Sizes whose product would not fit 64 bits are refused before it is formed.
    assert lib.kidi_attention_decode_static_need(2**31 - 1, 2**31 - 1, 2**31 - 1) == -1
    block.rows, block.heads, block.splits = 2**31 - 1, 2**31 - 1, 2**31 - 1
    assert lib.kidi_attention_decode_static(ctypes.byref(block), stream) == -3
    torch.cuda.synchronize()
