"""Each kernel alone against its plain reference, at sizes the engine's tiny models do
not have. Inputs are made so that faults show: one far key that must win among
hundreds, a key just outside a window, pages handed out in scrambled order."""
import math

import numpy as np
import pytest
import torch

import plain_model

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"


def close(found: torch.Tensor, expected: torch.Tensor, tolerance: float, what: str = ""):
    found, expected = found.double().cpu(), expected.double().cpu()
    scale = max(1.0, float(expected.abs().max()))
    error = float((found - expected).abs().max()) / scale
    assert error <= tolerance, f"{what}: relative error {error:.3e} > {tolerance:.1e}"


def bf16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(torch.float32)


# ------------------------------------------------------------------ embedding
@pytest.mark.parametrize("table_dtype", [torch.float32, torch.bfloat16])
def test_embedding(table_dtype):
    from kidi_b200.kernels import ops
    generator = torch.Generator().manual_seed(0)
    table = torch.randn(301, 200, generator=generator).to(table_dtype)
    tokens = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32)
    out = ops.embedding(tokens.to(DEVICE), table.to(DEVICE), 1.5)
    assert out.dtype == torch.float32
    assert torch.equal(out.cpu(), table.float()[tokens.long()] * 1.5)


# -------------------------------------------------------------------- rmsnorm
@pytest.mark.parametrize("hidden", [40, 1000, 1024, 3072, 4096, 5120, 7168, 8192, 9216])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(hidden, dtype):
    from kidi_b200.kernels import ops
    generator = torch.Generator().manual_seed(hidden)
    residual = torch.randn(7, hidden, generator=generator) * 3
    delta = (torch.randn(7, hidden, generator=generator)).to(dtype)
    weight = (1 + 0.1 * torch.randn(hidden, generator=generator)).to(dtype)
    eps = 1e-5
    device_residual = residual.to(DEVICE)
    out = ops.add_rmsnorm(device_residual, delta.to(DEVICE), weight.to(DEVICE), eps, dtype)
    summed = residual.double() + delta.double()
    expected = plain_model.rms_norm(summed, weight.double(), eps)
    close(device_residual, summed, 1e-6, "residual sum")
    close(out, expected, 1e-5 if dtype == torch.float32 else 8e-3, "normed")
    # Selected rows only, without a delta, leaving the stream untouched.
    rows = torch.tensor([6, 0, 3], dtype=torch.int32)
    before = device_residual.clone()
    picked = ops.add_rmsnorm(device_residual, None, weight.to(DEVICE), eps, torch.float32, row_index=rows.to(DEVICE))
    assert torch.equal(before, device_residual)
    close(picked, plain_model.rms_norm(before.cpu().double()[rows.long()], weight.double(), eps), 1e-5, "picked rows")


@pytest.mark.parametrize("dtype,inter", [(torch.float32, 136), (torch.bfloat16, 136), (torch.bfloat16, 201)])
def test_silu_gate(dtype, inter):
    from kidi_b200.kernels import ops
    generator = torch.Generator().manual_seed(1)
    gate_up = (torch.randn(37, 2 * inter, generator=generator) * 4).to(dtype)
    out = ops.silu_gate(gate_up.to(DEVICE))
    gate, up = gate_up[:, :inter].double(), gate_up[:, inter:].double()
    close(out, gate / (1 + torch.exp(-gate)) * up, 1e-6 if dtype == torch.float32 else 5e-3, "silu gate")


# ----------------------------------------------------------------------- gemm
@pytest.mark.parametrize("shape", [(1, 389, 96), (70, 130, 200), (129, 64, 17)])
def test_gemm_32_bit(shape):
    from kidi_b200.kernels import ops
    M, N, K = shape
    generator = torch.Generator().manual_seed(M)
    x, w = torch.randn(M, K, generator=generator), torch.randn(N, K, generator=generator)
    out = ops.gemm_simt(x.to(DEVICE), w.to(DEVICE), torch.float32)
    close(out, x.double() @ w.double().T, 2e-6, "gemm_simt")
    # A row's result does not depend on the rows around it.
    alone = ops.gemm_simt(x[M // 2:M // 2 + 1].to(DEVICE), w.to(DEVICE), torch.float32)
    assert torch.equal(alone[0], out[M // 2])


@pytest.mark.parametrize("rows", [1, 3, 8, 9, 16, 31, 64])
@pytest.mark.parametrize("shape", [(389, 96), (100, 200), (4096, 1024), (40, 4104)])
@pytest.mark.parametrize("row_tiles", [1, 2])
def test_gemm_skinny(rows, shape, row_tiles):
    from kidi_b200.kernels import skinny
    N, K = shape
    generator = torch.Generator().manual_seed(rows * 1000 + N)
    x = torch.randn(rows, K, generator=generator).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=generator) / math.sqrt(K)).to(torch.bfloat16)
    expected = x.double() @ w.double().T
    for out_dtype, tolerance in ((torch.float32, 2e-5), (torch.bfloat16, 5e-3)):
        out = skinny.gemm(x.to(DEVICE), w.to(DEVICE), out_dtype, row_tiles=row_tiles)
        assert out.dtype == out_dtype
        close(out, expected, tolerance, f"gemm_skinny {rows}x{N}x{K} -> {out_dtype}")


@pytest.mark.parametrize("rows", [1, 8, 13, 40])
def test_gemm_skinny_silu_gate(rows):
    from kidi_b200.kernels import skinny
    inter, K = 200, 96
    generator = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, K, generator=generator).to(torch.bfloat16)
    w = (torch.randn(2 * inter, K, generator=generator) / math.sqrt(K) * 2).to(torch.bfloat16)
    gate = x.double() @ w[:inter].double().T
    up = x.double() @ w[inter:].double().T
    out = skinny.gemm_silu_gate(x.to(DEVICE), w.to(DEVICE))
    close(out, gate / (1 + torch.exp(-gate)) * up, 5e-3, "fused silu gate")


@pytest.mark.parametrize("rows", [1, 8, 13, 40, 64, 100, 300])
@pytest.mark.parametrize("shape", [(389, 96), (100, 200), (4096, 1024), (130, 4104)])
@pytest.mark.parametrize("splits", [1, 3, None])
def test_gemm_tcgen05(rows, shape, splits):
    """The tensor-memory kernel: every tile size, ragged edges in all three dimensions,
    with and without split-K (whose partial sums are added in slice order)."""
    from kidi_b200.kernels import tcgen05
    N, K = shape
    generator = torch.Generator().manual_seed(rows * 1000 + N)
    x = torch.randn(rows, K, generator=generator).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=generator) / math.sqrt(K)).to(torch.bfloat16)
    expected = x.double() @ w.double().T
    for out_dtype, tolerance in ((torch.float32, 2e-5), (torch.bfloat16, 5e-3)):
        out = tcgen05.gemm(x.to(DEVICE), w.to(DEVICE), out_dtype, splits=splits)
        close(out, expected, tolerance, f"gemm_tcgen05 {rows}x{N}x{K} splits {splits} -> {out_dtype}")
        again = tcgen05.gemm(x.to(DEVICE), w.to(DEVICE), out_dtype, splits=splits)
        assert torch.equal(out, again)          # the sum over slices does not depend on timing
    assert tcgen05.error_code(torch.device(DEVICE)) == 0


@pytest.mark.parametrize("rows", [1, 17, 64, 150])
@pytest.mark.parametrize("splits", [1, 2])
def test_gemm_tcgen05_silu_gate(rows, splits):
    from kidi_b200.kernels import tcgen05
    inter, K = 200, 96
    generator = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, K, generator=generator).to(torch.bfloat16)
    w = (torch.randn(2 * inter, K, generator=generator) / math.sqrt(K) * 2).to(torch.bfloat16)
    gate = x.double() @ w[:inter].double().T
    up = x.double() @ w[inter:].double().T
    out = tcgen05.gemm_silu_gate(x.to(DEVICE), w.to(DEVICE), splits=splits)
    close(out, gate / (1 + torch.exp(-gate)) * up, 5e-3, "fused silu gate (tcgen05)")
    assert tcgen05.error_code(torch.device(DEVICE)) == 0


@pytest.mark.parametrize("rows", [1, 5, 8])
@pytest.mark.parametrize("shape", [(389, 96, 200), (4096, 1024, 520), (48, 4104, 64)])
@pytest.mark.parametrize("norm_dtype", [torch.bfloat16, torch.float32])
def test_the_norm_between_two_products_without_a_kernel_of_its_own(rows, shape, norm_dtype):
    """The product before an RMSNorm adds its result to the residual stream and leaves the rows
    times the norm's weight and the parts of their sums of squares; the product after applies
    each row's factor (plain and with the SiLU gate); `apply_row_factors` makes plain rows.
    Against the plain residual sum, norm and products in 64-bit."""
    from kidi_b200.kernels import ops, skinny
    N, K, N2 = shape
    eps = 1e-5
    generator = torch.Generator().manual_seed(rows * 7 + N)
    x = torch.randn(rows, K, generator=generator).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=generator) / math.sqrt(K)).to(torch.bfloat16)
    bias = torch.randn(N, generator=generator)
    residual = torch.randn(rows, N, generator=generator) * 2
    norm_weight = (1 + 0.1 * torch.randn(N, generator=generator)).to(norm_dtype)
    w2 = (torch.randn(2 * N2, N, generator=generator) / math.sqrt(N)).to(torch.bfloat16)
    summed = residual.double() + x.double() @ w.double().T + bias.double()
    normed = plain_model.rms_norm(summed, norm_weight.double(), eps)

    device_residual = residual.to(DEVICE)
    values, parts = skinny.gemm_into_residual(x.to(DEVICE), w.to(DEVICE), device_residual, norm_weight.to(DEVICE),
                                              bias=bias.to(DEVICE))
    assert values.shape == (rows, N) and parts.shape == (rows, -(-N // 16))
    close(device_residual, summed, 2e-5, "the residual stream after the product")
    close(parts.double().sum(dim=1), (summed * summed).sum(dim=1), 1e-5, "sums of squares")
    close(values, summed * norm_weight.double(), 5e-3, "rows times the norm's weight")
    close(ops.apply_row_factors(values, parts, N, eps), normed, 8e-3, "plain rows")
    factors = (parts, N, eps)
    if N % 8 == 0:
        expected = normed @ w2.double().T
        close(skinny.gemm(values, w2.to(DEVICE), torch.bfloat16, factors=factors), expected, 1e-2, "product with row factors")
        gate, up = expected[:, :N2], expected[:, N2:]
        close(skinny.gemm_silu_gate(values, w2.to(DEVICE), factors=factors), gate / (1 + torch.exp(-gate)) * up, 1e-2,
              "gated product with row factors")
        # A second product into the residual, fed with rows that lack their factor (as a layer's last
        # product is when it follows a prepared norm).
        back = (torch.randn(N, N, generator=generator) / math.sqrt(N)).to(torch.bfloat16)
        again_values, again_parts = skinny.gemm_into_residual(values, back.to(DEVICE), device_residual,
                                                              norm_weight.to(DEVICE), factors=factors)
        twice = summed + normed @ back.double().T
        close(device_residual, twice, 8e-3, "a product with row factors into the residual")
        close(again_parts.double().sum(dim=1), (twice * twice).sum(dim=1), 2e-2, "its sums of squares")


@pytest.mark.parametrize("rows,shape", [(1, (389, 96)), (8, (4096, 1024)), (13, (130, 200)), (300, (389, 96))])
def test_products_with_a_bias(rows, shape):
    """y = x W^T + b in every product kernel (the bias in 32-bit, added in the epilogue) and
    after a product of the vendor library."""
    from kidi_b200.kernels import ops, skinny, tcgen05
    N, K = shape
    generator = torch.Generator().manual_seed(rows + N)
    x = torch.randn(rows, K, generator=generator).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=generator) / math.sqrt(K)).to(torch.bfloat16)
    bias = torch.randn(N, generator=generator) * 3
    expected = x.double() @ w.double().T + bias.double()
    device_x, device_w, device_bias = x.to(DEVICE), w.to(DEVICE), bias.to(DEVICE)
    for out_dtype, tolerance in ((torch.float32, 2e-5), (torch.bfloat16, 5e-3)):
        close(ops.gemm_simt(device_x, device_w, out_dtype, bias=device_bias), expected, tolerance, "gemm_simt + bias")
        close(ops.gemm_simt(device_x.float(), device_w.float(), out_dtype, bias=device_bias), expected, tolerance,
              "gemm_simt in 32-bit + bias")
        if rows <= 64:
            close(skinny.gemm(device_x, device_w, out_dtype, bias=device_bias), expected, tolerance, "gemm_skinny + bias")
        close(tcgen05.gemm(device_x, device_w, out_dtype, bias=device_bias), expected, tolerance, "gemm_tcgen05 + bias")
        close(tcgen05.gemm(device_x, device_w, out_dtype, bias=device_bias, splits=2), expected, tolerance,
              "gemm_tcgen05 split + bias")
        product = (x.double() @ w.double().T).to(out_dtype).to(DEVICE)
        close(ops.add_bias(product, device_bias), expected, tolerance, "add_bias")
    with pytest.raises(Exception):
        ops.add_bias(product, device_bias[:-1])
    assert tcgen05.error_code(torch.device(DEVICE)) == 0


# ------------------------------------------------------ rope, cache, attention
class Tables:
    pass


def make_cache_and_tables(starts, news, kv_heads, head_dim, window, dtype, max_tokens=4096, scramble=True):
    """A cache with one entry, slots whose pages were handed out in a scrambled order,
    and the device tables of a step in which sequence b holds starts[b] tokens and
    brings news[b] more."""
    from kidi_b200.cache.sequence_cache import KVRequest, SequenceCache
    from kidi_b200.engine.plan import StepBatch, build_plan
    cache = SequenceCache([[KVRequest(kv_heads, head_dim, window)]], max_tokens=max_tokens, max_positions=2048,
                          dtype=dtype, device=torch.device(DEVICE))
    if scramble:  # take and give back pages so that the free list is out of order
        junk = [cache.acquire() for _ in range(5)]
        cache.reserve([(slot, 64 * (1 + index)) for index, slot in enumerate(junk)])
        for slot in junk[::2] + junk[1::2]:
            cache.release(slot)
    slots = [cache.acquire() for _ in starts]
    cache.reserve([(slot, start + new) for slot, start, new in zip(slots, starts, news)])
    cache.flush_tables()
    plan = build_plan(StepBatch(slots, [[0] * new for new in news]), starts, vocab_size=10)
    tables = Tables()
    for name in plan.FIELDS:
        setattr(tables, name, torch.from_numpy(getattr(plan, name)).to(DEVICE))
    return cache, slots, plan, tables


def gather_cache(view, slot_pages, length, ring_tokens=0):
    """[length, kv_heads, head_dim] keys and values of one sequence, read back through
    its page list (positions that a ring has overwritten come back as NaN)."""
    keys, values = view.keys.float().cpu(), view.values.float().cpu()
    page_size = view.page_size
    out_k = torch.full((length, keys.shape[1], keys.shape[3]), float("nan"))
    out_v = out_k.clone()
    for position in range(length):
        if ring_tokens and position < length - ring_tokens:
            continue
        index = position // page_size
        if ring_tokens:
            index %= ring_tokens // page_size
        page = slot_pages[index]
        out_k[position] = keys[page, :, position % page_size, :]
        out_v[position] = values[page, :, position % page_size, :]
    return out_k, out_v


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("geometry", [(5, 1, 80, 80), (3, 3, 16, 16), (4, 2, 256, 64)])
def test_rope_store(dtype, geometry):
    """Norm + rotation in place, and the rows land in the right pages."""
    from kidi_b200.kernels import ops
    heads, kv_heads, head_dim, rotary_dim = geometry
    starts, news = [0, 70, 3], [5, 1, 130]
    cache, slots, plan, tables = make_cache_and_tables(starts, news, kv_heads, head_dim, None, dtype)
    generator = torch.Generator().manual_seed(head_dim)
    width = (heads + 2 * kv_heads) * head_dim
    qkv = torch.randn(plan.n_rows, width, generator=generator).to(dtype)
    q_norm = 1 + 0.1 * torch.randn(head_dim, generator=generator)
    k_norm = 1 + 0.1 * torch.randn(head_dim, generator=generator)
    cos, sin = plain_model.rotary_tables(256, rotary_dim, 1e4)
    device_qkv = qkv.to(DEVICE)
    view = cache.views(0)[0]
    ops.rope_store(device_qkv, heads=heads, kv_heads=kv_heads, head_dim=head_dim, q_norm=q_norm.to(DEVICE),
                   k_norm=k_norm.to(DEVICE), eps=1e-6, cos=cos.to(DEVICE), sin=sin.to(DEVICE), rotary_dim=rotary_dim,
                   tables=tables, kv_view=view, store=True)
    positions = torch.from_numpy(plan.row_pos).long()
    x = qkv.double()
    q = x[:, :heads * head_dim].reshape(-1, heads, head_dim)
    k = x[:, heads * head_dim:(heads + kv_heads) * head_dim].reshape(-1, kv_heads, head_dim)
    v = x[:, (heads + kv_heads) * head_dim:].reshape(-1, kv_heads, head_dim)

    def expected_rotation(heads_tensor, weight):
        # Norm over the whole head, then rotation of its first rotary_dim elements.
        normed = plain_model.rms_norm(heads_tensor, weight.double(), 1e-6)
        half = rotary_dim // 2
        part = normed[..., :rotary_dim]
        turned = torch.cat([-part[..., half:], part[..., :half]], dim=-1)
        c = torch.cat([cos[positions], cos[positions]], dim=-1).double()[:, None, :]
        s = torch.cat([sin[positions], sin[positions]], dim=-1).double()[:, None, :]
        return torch.cat([part * c + turned * s, normed[..., rotary_dim:]], dim=-1)

    tolerance = 2e-6 if dtype == torch.float32 else 8e-3
    result = device_qkv.double().cpu()
    close(result[:, :heads * head_dim].reshape(-1, heads, head_dim), expected_rotation(q, q_norm), tolerance, "q")
    expected_k = expected_rotation(k, k_norm)
    close(result[:, heads * head_dim:(heads + kv_heads) * head_dim].reshape(-1, kv_heads, head_dim), expected_k,
          tolerance, "k in place")
    for index, slot in enumerate(slots):
        row0, new, start = int(plan.seq_row0[index]), news[index], starts[index]
        cached_k, cached_v = gather_cache(view, view.group.pages[slot], start + new)
        close(cached_k[start:], expected_k[row0:row0 + new], tolerance, f"cached keys of sequence {index}")
        close(cached_v[start:], v[row0:row0 + new], 1e-6 if dtype == torch.float32 else 8e-3, "cached values")
    cache.check()


def reference_attention(q, keys, values, positions, window, scale):
    """q [rows, heads, d] at `positions` of one sequence whose keys/values are [length, kv_heads, d]."""
    rows, heads, width = q.shape
    group = heads // keys.shape[1]
    out = torch.zeros(rows, heads, width, dtype=torch.float64)
    for row in range(rows):
        p = int(positions[row])
        first = max(0, p - window + 1) if window else 0
        for head in range(heads):
            k = keys[first:p + 1, head // group].double()
            v = values[first:p + 1, head // group].double()
            weights = torch.softmax((k @ q[row, head].double()) * scale, dim=0)
            out[row, head] = weights @ v
    return out.reshape(rows, heads * width)


class FakeContext:
    """What the attention launcher needs of a step."""

    def __init__(self, plan, tables):
        self.plan, self.tables = plan, tables
        self._held = {}

    def workspace(self, name, count, zero=False):
        if name not in self._held or self._held[name].numel() < count:
            self._held[name] = (torch.zeros if zero else torch.empty)(count, dtype=torch.float32, device=DEVICE)
        return self._held[name]


def launch_attention(kind, plan, tables, qkv, out, splits=None, ring=None, **arguments):
    from kidi_b200.kernels import attention, ops
    if kind == "generic":
        ops.attention_generic(qkv, out, tables=tables, **arguments)
    else:
        assert attention.fast_fits(qkv.dtype, arguments["heads"], arguments["kv_heads"], arguments["head_dim"],
                                   plan.is_decode and not arguments["keys_in_step"])
        # splits / ring None: the launcher's own choice of the decode kernel's form
        attention.run(FakeContext(plan, tables), qkv, out, splits=splits, ring=ring, **arguments)


@pytest.mark.parametrize("kind,dtype", [("generic", torch.float32), ("generic", torch.bfloat16),
                                        ("tensor_core", torch.bfloat16)])
@pytest.mark.parametrize("geometry", [(6, 2, 48, None), (4, 4, 128, None), (8, 1, 16, 37), (2, 1, 80, 100),
                                      (16, 2, 64, None), (3, 1, 256, 70)])
def test_attention_over_cache(kind, dtype, geometry):
    """Prompts of unequal length and single tokens against a cache filled by earlier
    steps, with one far key made to dominate."""
    from kidi_b200.kernels import ops
    heads, kv_heads, head_dim, window = geometry
    scale = 1.0 / math.sqrt(head_dim)
    starts, news = [300, 0, 129, 64], [1, 200, 1, 70]
    cache, slots, plan, tables = make_cache_and_tables(starts, news, kv_heads, head_dim, window, dtype)
    view = cache.views(0)[0]
    ring_tokens = view.ring_pages * view.page_size
    generator = torch.Generator().manual_seed(head_dim + heads)
    width = (heads + 2 * kv_heads) * head_dim
    history = {}
    # Earlier steps: write each sequence's first `start` keys and values through the kernel.
    for index, (slot, start) in enumerate(zip(slots, starts)):
        keys = torch.randn(start + news[index], kv_heads, head_dim, generator=generator)
        values = torch.randn(start + news[index], kv_heads, head_dim, generator=generator)
        if start > 150:  # a far key that one query direction loves
            keys[7] *= 0.0
            keys[7, :, 0] = 30.0
        history[index] = (keys.to(dtype).float(), values.to(dtype).float())
        if start == 0:
            continue
        from kidi_b200.engine.plan import StepBatch, build_plan
        earlier = build_plan(StepBatch([slot], [[0] * start]), [0], vocab_size=10)
        earlier_tables = Tables()
        for name in earlier.FIELDS:
            setattr(earlier_tables, name, torch.from_numpy(getattr(earlier, name)).to(DEVICE))
        packed = torch.zeros(start, width)
        packed[:, heads * head_dim:(heads + kv_heads) * head_dim] = keys[:start].reshape(start, -1)
        packed[:, (heads + kv_heads) * head_dim:] = values[:start].reshape(start, -1)
        ops.rope_store(packed.to(dtype).to(DEVICE), heads=heads, kv_heads=kv_heads, head_dim=head_dim, q_norm=None,
                       k_norm=None, eps=0.0, cos=None, sin=None, rotary_dim=0, tables=earlier_tables, kv_view=view,
                       store=True, transform=False)
    # This step's rows.
    qkv = torch.zeros(plan.n_rows, width)
    for index in range(len(slots)):
        row0, new, start = int(plan.seq_row0[index]), news[index], starts[index]
        keys, values = history[index]
        q = torch.randn(new, heads, head_dim, generator=generator)
        if start > 150:
            q[:, :, 0] = 4.0  # 4 * 30 / sqrt(d): the far key takes nearly all the weight when visible
        qkv[row0:row0 + new, :heads * head_dim] = q.reshape(new, -1)
        qkv[row0:row0 + new, heads * head_dim:(heads + kv_heads) * head_dim] = keys[start:].reshape(new, -1)
        qkv[row0:row0 + new, (heads + kv_heads) * head_dim:] = values[start:].reshape(new, -1)
    qkv = qkv.to(dtype)
    device_qkv = qkv.to(DEVICE)
    tolerance = 3e-6 if dtype == torch.float32 else 1e-2
    for keys_in_step in (True, False):
        if not keys_in_step:  # every key from the cache: store this step's rows first
            if ring_tokens and max(news) > 1:
                continue  # a ring is written after attention when a step brings several tokens
            ops.rope_store(device_qkv, heads=heads, kv_heads=kv_heads, head_dim=head_dim, q_norm=None, k_norm=None,
                           eps=0.0, cos=None, sin=None, rotary_dim=0, tables=tables, kv_view=view, store=True,
                           transform=False)
        out = torch.empty(plan.n_rows, heads * head_dim, dtype=dtype, device=DEVICE)
        launch_attention(kind, plan, tables, device_qkv, out, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                         scale=scale, window=window, kv_view=view, keys_in_step=keys_in_step)
        for index in range(len(slots)):
            row0, new, start = int(plan.seq_row0[index]), news[index], starts[index]
            keys, values = history[index]
            q = qkv[row0:row0 + new, :heads * head_dim].float().reshape(new, heads, head_dim)
            expected = reference_attention(q, keys, values, plan.row_pos[row0:row0 + new], window, scale)
            close(out[row0:row0 + new], expected, tolerance,
                  f"{kind}: sequence {index} (start {start}, new {new}, in step {keys_in_step})")


@pytest.mark.parametrize("kind,dtype", [("generic", torch.float32), ("tensor_core", torch.bfloat16)])
@pytest.mark.parametrize("geometry", [(8, 2, 128, None), (6, 6, 48, None), (16, 1, 32, 90), (4, 2, 64, 64),
                                      (4, 2, 256, None), (3, 1, 192, 100)])
@pytest.mark.parametrize("splits", [1, 3, 40])
def test_attention_decode(kind, dtype, geometry, splits):
    """One token per sequence against caches of very different lengths, with the key
    range split over several blocks; the far key at position 7 must be found."""
    from kidi_b200.engine.plan import StepBatch, build_plan
    from kidi_b200.kernels import ops
    if kind == "generic" and splits > 1:
        pytest.skip("the generic kernel does not split keys")
    heads, kv_heads, head_dim, window = geometry
    scale = 1.0 / math.sqrt(head_dim)
    starts = [0, 63, 64, 300, 1000, 127]
    if window:  # the loud key at position 7 is the last one inside the window, then the first one outside
        starts += [7 + window - 1, 7 + window]
    news = [1] * len(starts)
    cache, slots, plan, tables = make_cache_and_tables(starts, news, kv_heads, head_dim, window, dtype,
                                                       max_tokens=8192)
    view = cache.views(0)[0]
    generator = torch.Generator().manual_seed(head_dim * 7 + heads)
    width = (heads + 2 * kv_heads) * head_dim
    qkv = torch.zeros(len(starts), width)
    history = {}
    for index, (slot, start) in enumerate(zip(slots, starts)):
        total = start + 1
        keys = torch.randn(total, kv_heads, head_dim, generator=generator)
        values = torch.randn(total, kv_heads, head_dim, generator=generator)
        q = torch.randn(1, heads, head_dim, generator=generator)
        if total > 150 or index >= 6:
            keys[7] *= 0.0
            keys[7, :, 0] = 30.0
            q[:, :, 0] = 4.0
        history[index] = (keys.to(dtype).float(), values.to(dtype).float())
        writer = build_plan(StepBatch([slot], [[0] * total]), [0], vocab_size=10)
        writer_tables = Tables()
        for name in writer.FIELDS:
            setattr(writer_tables, name, torch.from_numpy(getattr(writer, name)).to(DEVICE))
        packed = torch.zeros(total, width)
        packed[:, heads * head_dim:(heads + kv_heads) * head_dim] = keys.reshape(total, -1)
        packed[:, (heads + kv_heads) * head_dim:] = values.reshape(total, -1)
        ops.rope_store(packed.to(dtype).to(DEVICE), heads=heads, kv_heads=kv_heads, head_dim=head_dim, q_norm=None,
                       k_norm=None, eps=0.0, cos=None, sin=None, rotary_dim=0, tables=writer_tables, kv_view=view,
                       store=True, transform=False)
        qkv[index, :heads * head_dim] = q.reshape(-1)
    qkv = qkv.to(dtype)
    out = torch.empty(len(starts), heads * head_dim, dtype=dtype, device=DEVICE)
    launch_attention(kind, plan, tables, qkv.to(DEVICE), out, splits=splits, heads=heads, kv_heads=kv_heads,
                     head_dim=head_dim, scale=scale, window=window, kv_view=view, keys_in_step=False)
    # 32-bit: a thousand keys are summed into one accumulator, each addition rounding at
    # 2^-24 of the running value; the rounding adds like a random walk.
    tolerance = 1e-5 if dtype == torch.float32 else 1e-2
    for index, start in enumerate(starts):
        keys, values = history[index]
        q = qkv[index:index + 1, :heads * head_dim].float().reshape(1, heads, head_dim)
        expected = reference_attention(q, keys, values, [start], window, scale)
        close(out[index:index + 1], expected, tolerance, f"{kind}: sequence of {start + 1} tokens, {splits} splits")
    if kind == "tensor_core" and head_dim % 64 == 0:
        # The ring form of the page-copying kernel (three tiles that take keys and values in
        # turn), which the launcher takes by itself only for large batches.
        from kidi_b200.kernels import attention
        assert attention.ring_available(head_dim)
        ring_out = torch.empty_like(out)
        launch_attention(kind, plan, tables, qkv.to(DEVICE), ring_out, splits=splits, ring=True, heads=heads,
                         kv_heads=kv_heads, head_dim=head_dim, scale=scale, window=window, kv_view=view,
                         keys_in_step=False)
        for index, start in enumerate(starts):
            keys, values = history[index]
            q = qkv[index:index + 1, :heads * head_dim].float().reshape(1, heads, head_dim)
            expected = reference_attention(q, keys, values, [start], window, scale)
            close(ring_out[index:index + 1], expected, tolerance, f"ring: sequence of {start + 1} tokens, {splits} splits")
        assert attention.timeout_flags() == 0
    if kind == "tensor_core" and splits == 3:
        # Three splits merge inside a thread-block cluster; the same splits merged through a
        # workspace in global memory must agree.
        from kidi_b200.kernels import attention
        assert attention.CLUSTER_SPLITS >= 3
        through_workspace = torch.empty_like(out)
        saved, attention.CLUSTER_SPLITS = attention.CLUSTER_SPLITS, 0
        try:
            launch_attention(kind, plan, tables, qkv.to(DEVICE), through_workspace, splits=splits, heads=heads,
                             kv_heads=kv_heads, head_dim=head_dim, scale=scale, window=window, kv_view=view,
                             keys_in_step=False)
        finally:
            attention.CLUSTER_SPLITS = saved
        close(out, through_workspace, 8e-3, "cluster merge against workspace merge")  # one bfloat16 step


@pytest.mark.parametrize("geometry", [(8, 2, 128, None), (4, 4, 64, None), (6, 1, 128, 200), (2, 2, 64, 130),
                                      (5, 5, 128, 64)])
def test_attention_prompts_tensor_memory(geometry):
    """The tcgen05 prompt kernel: packed prompts that start at position 0, of lengths on
    both sides of its 128-row tiles, with a far key that long sequences must find and a
    window whose edge falls inside a tile."""
    from kidi_b200.kernels import attention
    heads, kv_heads, head_dim, window = geometry
    scale = 1.0 / math.sqrt(head_dim)
    lengths = [300, 1, 128, 129, 700, 64]
    starts = [0] * len(lengths)
    cache, slots, plan, tables = make_cache_and_tables(starts, lengths, kv_heads, head_dim, window, torch.bfloat16,
                                                       max_tokens=8192)
    generator = torch.Generator().manual_seed(head_dim + heads)
    width = (heads + 2 * kv_heads) * head_dim
    qkv = torch.zeros(plan.n_rows, width)
    history = {}
    for index, length in enumerate(lengths):
        row0 = int(plan.seq_row0[index])
        keys = torch.randn(length, kv_heads, head_dim, generator=generator)
        values = torch.randn(length, kv_heads, head_dim, generator=generator)
        q = torch.randn(length, heads, head_dim, generator=generator)
        if length > 150:
            keys[7] *= 0.0
            keys[7, :, 0] = 30.0
            q[:, :, 0] = 4.0
        history[index] = (keys.to(torch.bfloat16).float(), values.to(torch.bfloat16).float())
        qkv[row0:row0 + length, :heads * head_dim] = q.reshape(length, -1)
        qkv[row0:row0 + length, heads * head_dim:(heads + kv_heads) * head_dim] = keys.reshape(length, -1)
        qkv[row0:row0 + length, (heads + kv_heads) * head_dim:] = values.reshape(length, -1)
    qkv = qkv.to(torch.bfloat16)
    device_qkv = qkv.to(DEVICE)
    out = torch.full((plan.n_rows, heads * head_dim), float("nan"), dtype=torch.bfloat16, device=DEVICE)
    assert attention.tensor_memory_fits(device_qkv, out, head_dim, heads, kv_heads)
    attention.prefill_tensor_memory(device_qkv, out, tables.seq_len, tables.seq_row0, plan.n_seqs, plan.max_new,
                                    heads=heads, kv_heads=kv_heads, head_dim=head_dim, scale=scale, window=window)
    torch.cuda.synchronize()
    assert attention.timeout_flags() == 0
    for index, length in enumerate(lengths):
        row0 = int(plan.seq_row0[index])
        keys, values = history[index]
        q = qkv[row0:row0 + length, :heads * head_dim].float().reshape(length, heads, head_dim)
        expected = reference_attention(q, keys, values, plan.row_pos[row0:row0 + length], window, scale)
        close(out[row0:row0 + length], expected, 1e-2, f"sequence {index} of {length} tokens")
    # The dispatcher takes this kernel for such a step and agrees with itself.
    again = torch.empty_like(out)
    launch_attention("tensor_core", plan, tables, device_qkv, again, heads=heads, kv_heads=kv_heads,
                     head_dim=head_dim, scale=scale, window=window, kv_view=cache.views(0)[0], keys_in_step=True)
    assert torch.equal(again, out)


@pytest.mark.parametrize("geometry", [(8, 2, 128, None, 128), (6, 6, 48, None, 32), (16, 2, 64, 90, 64),
                                      (4, 1, 32, None, 0), (2, 1, 256, None, 64), (6, 2, 192, 70, 192)])
@pytest.mark.parametrize("splits", [1, 3])
@pytest.mark.parametrize("norm_dtype", [torch.bfloat16, torch.float32])
def test_decode_with_the_rotation_inside(geometry, splits, norm_dtype):
    """One token per sequence, given to the attention kernel as the projection left it:
    the kernel's own norm, rotation and cache write against the separate kernel followed
    by the same attention, on two copies of a filled cache."""
    from kidi_b200.engine.plan import StepBatch, build_plan
    from kidi_b200.kernels import attention, ops
    heads, kv_heads, head_dim, window, rotary_dim = geometry
    scale = 1.0 / math.sqrt(head_dim)
    starts = [0, 63, 64, 300, 1000, 127]
    news = [1] * len(starts)
    generator = torch.Generator().manual_seed(head_dim * 11 + heads)
    width = (heads + 2 * kv_heads) * head_dim
    qkv = torch.randn(len(starts), width, generator=generator).to(torch.bfloat16).to(DEVICE)
    q_norm = (1 + 0.1 * torch.randn(head_dim, generator=generator)).to(norm_dtype).to(DEVICE)
    k_norm = (1 + 0.1 * torch.randn(head_dim, generator=generator)).to(norm_dtype).to(DEVICE)
    if rotary_dim:
        cos, sin = plain_model.rotary_tables(2048, rotary_dim, 1e4)
        cos, sin = cos.to(DEVICE), sin.to(DEVICE)
    else:
        cos = sin = None
    results = []
    forms = [(False, None), (True, None)] + ([(True, True)] if attention.ring_available(head_dim) else [])
    for fused, ring in forms:
        cache, slots, plan, tables = make_cache_and_tables(starts, news, kv_heads, head_dim, window, torch.bfloat16,
                                                           max_tokens=8192)
        view = cache.views(0)[0]
        filler = torch.Generator().manual_seed(5)
        view.keys.copy_(torch.randn(view.keys.shape, generator=filler).to(torch.bfloat16))
        view.values.copy_(torch.randn(view.values.shape, generator=filler).to(torch.bfloat16))
        rows = qkv.clone()
        out = torch.empty(len(starts), heads * head_dim, dtype=torch.bfloat16, device=DEVICE)
        common = dict(heads=heads, kv_heads=kv_heads, head_dim=head_dim)
        if fused:
            assert attention.fuses_rotation(plan, rows, kv_view=view, q_norm=q_norm, k_norm=k_norm, cos=cos, sin=sin,
                                            rotary_dim=rotary_dim, **common)
            rotation = dict(q_norm=q_norm, k_norm=k_norm, eps=1e-6, cos=cos, sin=sin, rotary_dim=rotary_dim, store=True)
        else:
            ops.rope_store(rows, q_norm=q_norm, k_norm=k_norm, eps=1e-6, cos=cos, sin=sin, rotary_dim=rotary_dim,
                           tables=tables, kv_view=view, store=True, **common)
            rotation = None
        attention.run(FakeContext(plan, tables), rows, out, scale=scale, window=window, kv_view=view,
                      keys_in_step=False, rotation=rotation, splits=splits, ring=ring, **common)
        torch.cuda.synchronize()
        results.append((out, view.keys.clone(), view.values.clone(), [view.group.pages[slot] for slot in slots]))
    plain_out, plain_keys, plain_values, plain_pages = results[0]
    for fused_out, fused_keys, fused_values, fused_pages in results[1:]:       # the usual form, then the ring
        assert plain_pages == fused_pages
        assert torch.equal(fused_keys, plain_keys), "the keys written by the attention kernel differ from the separate kernel's"
        assert torch.equal(fused_values, plain_values)
        assert torch.isfinite(fused_out.float()).all()
        close(fused_out, plain_out, 8e-3, "attention with the rotation inside")      # one bfloat16 step
    assert attention.timeout_flags() == 0


def test_window_edge():
    """The key just outside the window must not be seen, the one just inside must."""
    from kidi_b200.kernels import ops
    heads = kv_heads = 1
    head_dim, window, length = 16, 10, 40
    cache, slots, plan, tables = make_cache_and_tables([0], [length], kv_heads, head_dim, window, torch.float32)
    qkv = torch.zeros(length, 3 * head_dim)
    qkv[:, 0] = 1.0                                   # every query looks along axis 0
    qkv[:, 2 * head_dim] = torch.arange(length).float()  # value = the key's position
    loud = 20
    qkv[loud, head_dim] = 200.0                       # key 20 drowns every other key while it is visible
    out = torch.empty(length, head_dim, device=DEVICE)
    ops.attention_generic(qkv.to(DEVICE), out, heads=1, kv_heads=1, head_dim=head_dim, scale=1.0, window=window,
                          tables=tables, kv_view=cache.views(0)[0], keys_in_step=True)
    seen = out[:, 0].cpu()
    for position in range(length):
        if loud <= position < loud + window:
            assert abs(float(seen[position]) - loud) < 1e-4, position
        else:
            first = max(0, position - window + 1)
            assert abs(float(seen[position]) - (first + position) / 2) < 1e-4, position


# ------------------------------------------------------------------- sampling
def test_argmax_rules():
    from kidi_b200.kernels import ops
    logits = torch.randn(6, 1000, generator=torch.Generator().manual_seed(2))
    logits[0, 17] = logits[0, 900] = 50.0        # a tie: the lowest index wins
    logits[1, 5] = float("nan")                  # NaN: invalid
    logits[2, 999] = float("inf")                # +inf: invalid
    logits[3, :] = float("-inf")                 # nothing finite: invalid
    logits[4, 999] = 60.0                        # the last element
    found = ops.argmax(logits.to(DEVICE)).cpu().tolist()
    assert found == [17, -1, -1, -1, 999, int(logits[5].argmax())]
    assert found == [plain_model.greedy_token(row.numpy()) for row in logits]
    # A wide vocabulary is scanned in slices by many blocks: the same rules across slice borders.
    wide = torch.randn(6, 151936, generator=torch.Generator().manual_seed(3))
    wide[0, 4747] = wide[0, 4748] = wide[0, 150000] = 50.0      # a tie across two slices
    wide[1, 100000] = float("nan")
    wide[2, 151935] = float("inf")
    wide[3, :] = float("-inf")
    wide[4, 151935] = 60.0
    found = ops.argmax(wide.to(DEVICE)).cpu().tolist()
    assert found == [4747, -1, -1, -1, 151935, int(wide[5].argmax())]


@pytest.mark.parametrize("vocab", [389, 151936])
def test_temperature_sampling(vocab):
    from kidi_b200.kernels import ops
    rows = 64
    generator = torch.Generator().manual_seed(vocab)
    logits = torch.randn(rows, vocab, generator=generator) * 3
    temperature = torch.full((rows,), 0.8)
    temperature[::8] = 0.0                       # greedy rows among sampled ones
    keys = torch.arange(rows, dtype=torch.int64) * 7 + 1
    steps = torch.arange(rows, dtype=torch.int32) % 5
    found = ops.sample(logits.to(DEVICE), temperature.to(DEVICE), 1234, keys.to(DEVICE), steps.to(DEVICE)).cpu()
    again = ops.sample(logits.to(DEVICE), temperature.to(DEVICE), 1234, keys.to(DEVICE), steps.to(DEVICE)).cpu()
    assert torch.equal(found, again)
    mismatches = 0
    for row in range(rows):
        expected = plain_model.temperature_token(logits[row].numpy(), float(temperature[row]), 1234, int(keys[row]),
                                                 int(steps[row]))
        if int(found[row]) != expected:
            # Only a draw that falls within rounding of a boundary of the cumulative
            # distribution may land on the neighbouring token.
            values = logits[row].double().numpy()
            weights = np.exp((values - values.max()) / float(temperature[row]))
            cumulative = np.cumsum(weights) / weights.sum()
            u = plain_model.uniform_number(1234, int(keys[row]), int(steps[row]))
            token = int(found[row])
            low = cumulative[token - 1] if token else 0.0
            assert low - 1e-5 <= u <= cumulative[token] + 1e-5, (row, token, expected)
            mismatches += 1
    assert mismatches <= 2
    # The draws follow the distribution: a peaked row is sampled at its peak most of the time.
    peaked = torch.zeros(512, vocab)
    peaked[:, 123] = 8.0
    draws = ops.sample(peaked.to(DEVICE), torch.ones(512, device=DEVICE), 7,
                       torch.arange(512, dtype=torch.int64, device=DEVICE),
                       torch.zeros(512, dtype=torch.int32, device=DEVICE)).cpu()
    share = float((draws == 123).float().mean())
    expected_share = math.exp(8.0) / (math.exp(8.0) + vocab - 1)
    assert abs(share - expected_share) < 0.08
