"""Each kernel alone against a plain PyTorch float32 reference of the same operation, at sizes
other than the engine's (odd widths, head sizes in steps of 16, vocabularies that are no power
of two), and with inputs made so that a fault would show."""

import math

import pytest
import torch

from miniserve_b200 import ops
from miniserve_b200.ops import attention_bf16, native
from tests.kernel_util import PagedBatch, make_context, reference_attention
from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu


def native_launches() -> int:
    from miniserve_b200.ops import native

    return native.LAUNCHES[0]
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


def _tol(dtype):
    return dict(atol=2e-6, rtol=2e-6) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden, vocab, tokens", [(24, 77, 5), (27, 50, 9), (1000, 333, 130)])
def test_embed_gather(dtype, hidden, vocab, tokens):
    table = torch.randn(vocab, hidden, device=DEV).to(dtype)
    ids = torch.randint(0, vocab, (tokens,), device=DEV, dtype=torch.int32)
    ids[0], ids[-1] = vocab - 1, 0
    out = torch.empty(tokens, hidden, device=DEV)
    ops.embed_gather(out, table, ids)
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden, rows, eps", [(24, 3, 1e-5), (1000, 37, 1e-6), (4100, 2, 1e-3)])
def test_add_rmsnorm(dtype, hidden, rows, eps):
    res = torch.randn(rows, hidden, device=DEV) * 3
    delta = (torch.randn(rows, hidden, device=DEV)).to(dtype)
    w = (1 + 0.1 * torch.randn(hidden, device=DEV)).to(dtype)
    total = res + delta.float()
    expect = total * torch.rsqrt((total * total).mean(-1, keepdim=True) + eps) * w.float()
    got_res = res.clone()
    out = torch.empty(rows, hidden, device=DEV, dtype=dtype)
    ops.add_rmsnorm(out, got_res, delta, w, eps)
    assert torch.allclose(got_res, total, atol=1e-6)  # the sum is stored back
    assert torch.allclose(out.float(), expect, **_tol(dtype))
    # without an addend the residual is left alone
    out2 = torch.empty_like(out)
    keep = res.clone()
    ops.add_rmsnorm(out2, keep, None, w, eps)
    assert torch.equal(keep, res)
    e2 = res * torch.rsqrt((res * res).mean(-1, keepdim=True) + eps) * w.float()
    assert torch.allclose(out2.float(), e2, **_tol(dtype))
    # gathered rows: only those rows, residual untouched
    idx = torch.tensor([rows - 1, 0], device=DEV, dtype=torch.int32)
    out3 = torch.full((2, hidden), float("nan"), device=DEV, dtype=dtype)
    keep = res.clone()
    ops.add_rmsnorm(out3, keep, delta, w, eps, rows=idx)
    assert torch.equal(keep, res)
    assert torch.allclose(out3.float(), expect[idx.long()], **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens, inter", [(3, 7), (65, 224), (9, 3072)])
def test_silu_mul(dtype, tokens, inter):
    gu = (torch.randn(tokens, 2 * inter, device=DEV) * 3).to(dtype)
    out = torch.empty(tokens, inter, device=DEV, dtype=dtype)
    ops.silu_mul(out, gu)
    g, u = gu[:, :inter].float(), gu[:, inter:].float()
    assert torch.allclose(out.float(), g * torch.sigmoid(g) * u, **_tol(dtype))


@pytest.mark.parametrize("m, n, k", [(1, 5, 3), (7, 503, 96), (130, 70, 129), (64, 64, 16)])
def test_gemm_f32_is_true_32bit_and_row_independent(m, n, k):
    a = torch.randn(m, k, device=DEV)
    w = torch.randn(n, k, device=DEV)
    out = ops.linear(a, w)
    expect = (a.double() @ w.double().T)
    assert (out.double() - expect).abs().max().item() < 1e-4 * math.sqrt(k)
    # far tighter than a reduced-precision (tf32/bf16 input) product could be
    assert (out.double() - expect).abs().max().item() < 0.05 * (a.bfloat16().double() @ w.bfloat16().double().T - expect).abs().max().item() + 1e-6
    # a row's result does not depend on the rows beside it
    alone = ops.linear(a[m // 2:m // 2 + 1].contiguous(), w)
    assert torch.equal(alone[0], out[m // 2])


@pytest.mark.parametrize("m, n, k", [(128, 128, 64), (17, 200, 72), (333, 1000, 1000), (2048, 1024, 2048), (130, 503, 96), (4096, 6144, 256)])
@pytest.mark.parametrize("epilogue", ["bf16", "f32", "silu_mul"])
@pytest.mark.parametrize("config", [0, 5, 10, 11, 20, 21], ids=["by_shape", "tile_per_cta", "persistent_256", "persistent_128", "two_cta_256", "two_cta_128"])
def test_tcgen05_gemm(m, n, k, epilogue, config):
    """config: 0 chosen from the shape; 5 one CTA per tile; 10 and 11 the persistent kernel (tiles of 256 and 128 columns) whose ring
    of stages runs on from tile to tile and whose two accumulators take turns; 20 the same with pairs of CTAs on 256 x 256 tiles."""
    from miniserve_b200.ops import native

    if config in (11, 21) and epilogue != "bf16":
        pytest.skip("the 128-column persistent tile is built for the plain bfloat16 epilogue only")
    torch.manual_seed(m + n)
    x = torch.randn(m, k, device=DEV).bfloat16()
    if epilogue == "silu_mul":
        w = (torch.randn(2 * n, k, device=DEV) / 8).bfloat16()
        g, u = x.float() @ w[:n].float().T, x.float() @ w[n:].float().T
        expect = g * torch.sigmoid(g) * u
        out = torch.full((m, n), float("nan"), device=DEV, dtype=torch.bfloat16)
    else:
        w = torch.randn(n, k, device=DEV).bfloat16()
        expect = x.float() @ w.float().T
        out = torch.full((m, n), float("nan"), device=DEV, dtype=torch.float32 if epilogue == "f32" else torch.bfloat16)
    native.gemm_tc().ms_gemm_tc_set_config(config)
    try:
        ops.linear_tc(x, w, out, epilogue)
        torch.cuda.synchronize()
    finally:
        native.gemm_tc().ms_gemm_tc_set_config(0)
    assert ops.device_status(DEV).item() == 0
    scale = expect.abs().max().item()
    tol = 1e-4 * scale if epilogue == "f32" else 8e-3 * scale
    assert (out.float() - expect).abs().max().item() <= tol


def test_bf16_linear_accumulates_in_float32():
    a = torch.randn(33, 520, device=DEV).bfloat16()
    w = torch.randn(77, 520, device=DEV).bfloat16()
    expect = a.float() @ w.float().T
    out32 = torch.empty(33, 77, device=DEV)
    ops.linear(a, w, out=out32)
    assert torch.allclose(out32, expect, atol=1e-3, rtol=1e-3)
    assert torch.allclose(ops.linear(a, w).float(), expect, atol=0.3, rtol=2e-2)


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("n, k", [(16, 32), (503, 96), (1000, 1024), (72, 3072), (151936, 64), (40000, 1024), (33333, 264),
                                  (20008, 3072), (19000, 4096)])
def test_skinny_gemm_bf16(m, n, k):
    torch.manual_seed(m * 1000 + n)
    x = torch.randn(m, k, device=DEV).bfloat16()
    w = torch.randn(n, k, device=DEV).bfloat16()
    expect = x.float() @ w.float().T
    tol = dict(atol=2e-3 * (k ** 0.5), rtol=2e-3)
    out32 = torch.full((m, n), float("nan"), device=DEV)
    ops.linear(x, w, out=out32)
    assert torch.allclose(out32, expect, **tol)
    out16 = ops.linear(x, w)
    assert out16.dtype == torch.bfloat16 and torch.allclose(out16.float(), expect, atol=0.05 * (k ** 0.5), rtol=2e-2)
    # a row's result does not depend on the rows beside it (where both shapes go to this kernel:
    # with k beyond 3,072 more than 8 rows go to the library)
    if ops._skinny_ok(x, w):
        alone = torch.empty(1, n, device=DEV)
        ops.linear(x[m - 1:m].contiguous(), w, out=alone)
        assert torch.equal(alone[0], out32[m - 1])
    # very wide outputs go to the kernel whose CTAs walk many row tiles: the same bits as one tile per CTA
    k_lib = native.kernels()
    k_lib.ms_gemm_skinny_set_stream(0)
    try:
        one_tile = torch.full((m, n), float("nan"), device=DEV)
        ops.linear(x, w, out=one_tile)
    finally:
        k_lib.ms_gemm_skinny_set_stream(1)
    assert torch.equal(one_tile, out32)


@pytest.mark.parametrize("m", [1, 7, 16, 17, 32, 33, 64])
@pytest.mark.parametrize("n, k", [(1024, 3072), (4096, 12288), (1000, 2056), (130, 264), (77, 25600), (6144, 4096)])
def test_tcgen05_decode_product_with_swapped_operands(m, n, k):
    """The decode product on the tensor cores (the weight's rows as the instruction's M, k cut into the CTAs
    of a cluster) against float32 matmul, at widths and k that are no multiples of its tiles; a row's
    result does not depend on the rows beside it."""
    torch.manual_seed(m * 1000 + n)
    x = torch.randn(m, k, device=DEV).bfloat16()
    w = (torch.randn(n, k, device=DEV) * k ** -0.5).bfloat16()
    out = torch.full((m, n), float("nan"), device=DEV, dtype=torch.bfloat16)
    ops.linear_tc_decode(x, w, out)
    torch.cuda.synchronize()
    assert ops.device_status(DEV).item() == 0
    expect = x.float() @ w.float().T
    assert torch.allclose(out.float(), expect, atol=2e-2, rtol=2e-2)
    alone = torch.empty(1, n, device=DEV, dtype=torch.bfloat16)
    ops.linear_tc_decode(x[m - 1:m].contiguous(), w, alone)
    assert torch.equal(alone[0], out[m - 1])
    # and linear() sends the long and narrow ones of up to 32 rows here (a single row only beyond the register-fed kernel's k)
    if m <= 32 and k >= 2 * n and k >= 2048 and (m >= 2 or k > 3072):
        assert ops._tc_decode_ok(x, w, None) and torch.equal(ops.linear(x, w), out)


@pytest.mark.parametrize("m, inter, k", [(1, 3072, 1024), (8, 3072, 1024), (13, 224, 96), (16, 136, 64), (5, 2048, 4096)])
def test_skinny_gate_up_with_the_activation_in_its_epilogue(m, inter, k):
    """One kernel for silu(x Wg^T) * (x Wu^T) at decode sizes: the same numbers as the product into a
    [M, 2I] tensor followed by the activation kernel (both round the products to bfloat16 first)."""
    torch.manual_seed(m + inter)
    x = torch.randn(m, k, device=DEV).bfloat16()
    w = (torch.randn(2 * inter, k, device=DEV) * k ** -0.5).bfloat16()
    gate_up = ops.linear(x, w)
    want = torch.empty(m, inter, device=DEV, dtype=torch.bfloat16)
    ops.silu_mul(want, gate_up)
    got = torch.full((m, inter), float("nan"), device=DEV, dtype=torch.bfloat16)
    before = native_launches()
    ops.linear_silu_mul(x, w, got)
    assert native_launches() - before == 1
    assert torch.equal(got, want)
    ref = torch.nn.functional.silu(x.float() @ w[:inter].float().t()) * (x.float() @ w[inter:].float().t())
    assert torch.allclose(got.float(), ref, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq, nkv, d, page, theta, eps", [(4, 2, 16, 16, 1e4, 1e-6), (6, 1, 48, 8, 1e6, 1e-5),
                                                        (3, 3, 80, 4, 5e5, 1e-6), (2, 1, 256, 32, 1e6, 1e-6),
                                                        (16, 8, 128, 16, 1e6, 1e-6), (5, 5, 128, 8, 1e4, 1e-5)])
def test_qk_norm_rope_kv_write(dtype, nq, nkv, d, page, theta, eps):
    rows = [(0, 9), (13, 1), (30, 6)]  # a fresh portion, a decode token, a portion across a page edge
    pb = PagedBatch(rows, page, nkv, d, dtype, seed=3)
    t = pb.num_tokens
    qkv = torch.randn(t, (nq + 2 * nkv) * d, device=DEV).to(dtype)
    qw = (1 + 0.1 * torch.randn(d, device=DEV)).to(dtype)
    kw = (1 + 0.1 * torch.randn(d, device=DEV)).to(dtype)
    inv_freq = (1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))).to(DEV)
    q_out = torch.empty(t, nq, d, device=DEV, dtype=dtype)
    ops.qk_norm_rope_kv(q_out, pb.k_pool, pb.v_pool, qkv, qw, kw, inv_freq, d, eps, pb.positions, pb.row_of_token,
                        pb.page_indptr, pb.page_indices, page, pb.status)
    assert pb.status.item() == 0
    # plain float32 reference of the same operation
    x = qkv.float().cpu()
    q, k, v = x[:, :nq * d].view(t, nq, d), x[:, nq * d:(nq + nkv) * d].view(t, nkv, d), x[:, (nq + nkv) * d:].view(t, nkv, d)
    cos, sin = plain.rope_cos_sin(pb.positions.cpu(), d, theta, torch.float32)
    q_ref = plain.apply_rope(plain.rms_norm(q, qw.float().cpu(), eps), cos, sin)
    k_ref = plain.apply_rope(plain.rms_norm(k, kw.float().cpu(), eps), cos, sin)
    tol = dict(atol=5e-6, rtol=1e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
    assert torch.allclose(q_out.float().cpu(), q_ref, **tol)
    at = 0
    written = torch.zeros(pb.num_pages, page, dtype=torch.bool)
    for r, (s, n) in enumerate(rows):
        for i in range(n):
            p = s + i
            pg = pb.tables[r][p // page]
            written[pg, p % page] = True
            assert torch.allclose(pb.k_pool[pg, :, p % page].float().cpu(), k_ref[at], **tol)
            assert torch.equal(pb.v_pool[pg, :, p % page].float().cpu(), v[at])
            at += 1
    # nothing but the new tokens' slots was written (the pool was NaN before)
    assert torch.equal(~torch.isnan(pb.k_pool[:, 0, :, 0]).cpu(), written)


@pytest.mark.parametrize("nq, nkv, page, rotate, normed", [(16, 8, 16, True, True), (4, 2, 8, True, False), (2, 2, 64, False, True),
                                                          (6, 4, 16, True, True)])
@pytest.mark.parametrize("rows", [[(0, 300), (13, 1), (500, 213)], [(0, 1000)], [(3, 129), (0, 127), (40, 2), (0, 70)]])
def test_qkv_product_with_norm_rotation_and_cache_write_in_its_epilogue(nq, nkv, page, rotate, normed, rows):
    """The 2-CTA tcgen05 kernel's q|k|v epilogue against the product followed by the separate kernel:
    the same q, the same new keys and values in the same slots, nothing else touched."""
    d, hidden, eps = 128, 256, 1e-6
    torch.manual_seed(nq * 100 + len(rows))
    a = PagedBatch(rows, page, nkv, d, torch.bfloat16, seed=3)
    b = PagedBatch(rows, page, nkv, d, torch.bfloat16, seed=3)
    t = a.num_tokens
    x = torch.randn(t, hidden, device=DEV).bfloat16()
    w = (torch.randn((nq + 2 * nkv) * d, hidden, device=DEV) * hidden ** -0.5).bfloat16()
    qw = (1 + 0.1 * torch.randn(d, device=DEV)).bfloat16() if normed else None
    kw = (1 + 0.1 * torch.randn(d, device=DEV)).bfloat16() if normed else None
    inv_freq = (1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))).to(DEV) if rotate else None
    table = ops.rope_table(a.positions, inv_freq, t, d) if rotate else None
    q1 = torch.full((t, nq, d), float("nan"), device=DEV, dtype=torch.bfloat16)
    q2 = torch.full_like(q1, float("nan"))
    ops.qk_norm_rope_kv(q1, a.k_pool, a.v_pool, ops.linear(x, w), qw, kw, inv_freq, d if rotate else 0, eps, a.positions, a.row_of_token,
                        a.page_indptr, a.page_indices, page, a.status, cos_sin=table)
    tiled = None
    if rotate:
        # the epilogue reads the table by tiles of 128 tokens and eighths of the 64 pairs
        tiled = ops.rope_table_tiled(table)
        padded = torch.zeros((tiled.shape[0] * 128, 128), device=DEV)
        padded[:t] = table
        want = padded.view(-1, 128, 2, 8, 8).permute(0, 3, 2, 1, 4)  # [tile, eighth, cos|sin, token, pair]
        live = torch.arange(tiled.shape[0] * 128, device=DEV).view(-1, 1, 1, 128, 1).expand_as(want) < t
        assert torch.equal(torch.where(live, tiled, 0), torch.where(live, want, 0))
    ops.qkv_norm_rope_kv(q2, b.k_pool, b.v_pool, x, w, qw, kw, tiled, eps, b.positions, b.row_of_token, b.page_indptr, b.page_indices, page)
    torch.cuda.synchronize()
    assert a.status.item() == 0 and ops.device_status(DEV).item() == 0
    tol = dict(atol=3e-2, rtol=2e-2)
    assert torch.allclose(q2.float(), q1.float(), **tol)
    # the pools: NaN (never written) in the same places, close values in the others, values bit-equal
    for p1, p2, exact in ((a.k_pool, b.k_pool, False), (a.v_pool, b.v_pool, True)):
        assert torch.equal(torch.isnan(p1), torch.isnan(p2))
        x1, x2 = torch.nan_to_num(p1.float()), torch.nan_to_num(p2.float())
        assert torch.equal(x1, x2) if exact else torch.allclose(x2, x1, **tol)
    assert (~torch.isnan(b.k_pool[:, 0, :, 0])).sum().item() == t


def test_rope_angles_at_far_positions_are_32bit():
    d, theta, page = 32, 1e6, 16
    pb = PagedBatch([(40000, 3)], page, 1, d, torch.float32)
    qkv = torch.randn(3, 3 * d, device=DEV)
    inv_freq = (1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))).to(DEV)
    q_out = torch.empty(3, 1, d, device=DEV)
    ops.qk_norm_rope_kv(q_out, pb.k_pool, pb.v_pool, qkv, None, None, inv_freq, d, 0.0, pb.positions, pb.row_of_token,
                        pb.page_indptr, pb.page_indices, page, pb.status)
    cos, sin = plain.rope_cos_sin(pb.positions.cpu(), d, theta, torch.float32)
    ref = plain.apply_rope(qkv[:, :d].view(3, 1, d).cpu(), cos, sin)
    assert torch.allclose(q_out.cpu(), ref, atol=2e-5)


def _attention_case(dtype, rows, nq, nkv, d, page, window=None, needle=None, seed=0):
    torch.manual_seed(seed)
    pb = PagedBatch(rows, page, nkv, d, dtype, seed=seed)
    qs, refs = [], []
    scale = d ** -0.5
    for r, (s, n) in enumerate(rows):
        k = torch.randn(s + n, nkv, d, device=DEV).to(dtype)
        v = torch.randn(s + n, nkv, d, device=DEV).to(dtype)
        q = torch.randn(n, nq, d, device=DEV).to(dtype)
        if needle is not None and s + n > needle:
            # one far key that the last query must find: its score (16 * sqrt(d)) stands out from the
            # others (about +-4 * 3.5), and its value is unlike the rest
            q[-1] = 4.0
            k[needle] = 4.0
            v[needle] = 50.0
        pb.fill(r, k, v)
        qs.append(q)
        refs.append(reference_attention(q, k, v, list(range(s, s + n)), scale, window))
    q_all = torch.cat(qs).contiguous()
    return pb, q_all, torch.cat(refs), scale


ATT_SHAPES = [(4, 2, 16, 16), (6, 1, 32, 8), (8, 8, 48, 4), (16, 8, 128, 16), (5, 5, 80, 32), (2, 1, 256, 16)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq, nkv, d, page", ATT_SHAPES)
def test_attention_rowwise_mixed_batch(dtype, nq, nkv, d, page):
    rows = [(0, 37), (52, 1), (15, 18), (0, 1), (63, 2)]
    pb, q, ref, scale = _attention_case(dtype, rows, nq, nkv, d, page)
    out = torch.empty_like(q)
    ops.attention_rowwise(out, q, pb.k_pool, pb.v_pool, pb.positions, pb.row_of_token, pb.page_indptr,
                          pb.page_indices, scale, None, pb.status)
    assert pb.status.item() == 0
    tol = dict(atol=3e-6, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    assert torch.allclose(out.float(), ref, **tol)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_rowwise_finds_a_far_key_among_hundreds(dtype):
    rows = [(700, 1), (0, 650)]
    pb, q, ref, scale = _attention_case(dtype, rows, 4, 2, 64, 16, needle=3)
    out = torch.empty_like(q)
    ops.attention_rowwise(out, q, pb.k_pool, pb.v_pool, pb.positions, pb.row_of_token, pb.page_indptr,
                          pb.page_indices, scale, None, pb.status)
    assert ref[0, 0].mean().item() > 40  # the needle dominates the decode row's head 0
    tol = dict(atol=2e-4, rtol=1e-5) if dtype == torch.float32 else dict(atol=0.3, rtol=2e-2)
    assert torch.allclose(out.float(), ref, **tol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 7, 16, 33])
def test_attention_rowwise_window_edge(dtype, window):
    rows = [(0, 50), (49, 1)]
    pb, q, ref, scale = _attention_case(dtype, rows, 4, 2, 32, 8, window=window)
    out = torch.empty_like(q)
    ops.attention_rowwise(out, q, pb.k_pool, pb.v_pool, pb.positions, pb.row_of_token, pb.page_indptr,
                          pb.page_indices, scale, window, pb.status)
    tol = dict(atol=3e-6, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    assert torch.allclose(out.float(), ref, **tol)


def test_attention_rowwise_is_bit_identical_across_batching():
    nq, nkv, d, page = 6, 2, 48, 8
    torch.manual_seed(4)
    n = 77
    k = torch.randn(n, nkv, d, device=DEV)
    v = torch.randn(n, nkv, d, device=DEV)
    q = torch.randn(n, nq, d, device=DEV)

    def run(rows_spec, seed):
        pb = PagedBatch(rows_spec, page, nkv, d, torch.float32, seed=seed)
        qs = []
        for r, (s, cnt) in enumerate(rows_spec):
            pb.fill(r, k[:s + cnt], v[:s + cnt])
            qs.append(q[s:s + cnt])
        qq = torch.cat(qs).contiguous()
        out = torch.empty_like(qq)
        ops.attention_rowwise(out, qq, pb.k_pool, pb.v_pool, pb.positions, pb.row_of_token, pb.page_indptr,
                              pb.page_indices, d ** -0.5, None, pb.status)
        return out

    whole = run([(0, n)], 0)
    parts = run([(60, 17), (0, 5), (5, 55)], 9)  # other pages, other neighbours, other order
    assert torch.equal(parts[:17], whole[60:]) and torch.equal(parts[17:22], whole[:5]) and torch.equal(parts[22:], whole[5:60])


def test_attention_reports_a_page_that_was_given_back():
    pb, q, _, scale = _attention_case(torch.float32, [(0, 20)], 2, 1, 16, 8)
    pb.page_indices[0] = -1
    out = torch.empty_like(q)
    ops.attention_rowwise(out, q, pb.k_pool, pb.v_pool, pb.positions, pb.row_of_token, pb.page_indptr,
                          pb.page_indices, scale, None, pb.status)
    assert pb.status.item() != 0


# ------------------------------------------------------------------ bfloat16 tensor-core attention
BF16_TOL = dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("nq, nkv, d, page", ATT_SHAPES + [(8, 2, 64, 64), (32, 1, 16, 16)])
def test_attention_bf16_prompts_and_mixed_steps(nq, nkv, d, page):
    rows = [(0, 37), (52, 1), (15, 18), (0, 1), (63, 2), (0, 150), (100, 70), (64, 64)]
    pb, q, ref, scale = _attention_case(torch.bfloat16, rows, nq, nkv, d, page)
    out = torch.full_like(q, float("nan"))
    attention_bf16.run(out, q, pb.k_pool, pb.v_pool, make_context(pb), 0, scale, None)
    assert torch.allclose(out.float(), ref, **BF16_TOL)


@pytest.mark.parametrize("window", [1, 7, 64, 65, 100])
def test_attention_bf16_prompt_window_edge(window):
    rows = [(0, 200), (130, 3), (199, 1)]
    pb, q, ref, scale = _attention_case(torch.bfloat16, rows, 4, 2, 32, 8, window=window)
    out = torch.full_like(q, float("nan"))
    attention_bf16.run(out, q, pb.k_pool, pb.v_pool, make_context(pb), 0, scale, window)
    assert torch.allclose(out.float(), ref, **BF16_TOL)


@pytest.mark.parametrize("nq, nkv, d, page", ATT_SHAPES + [(8, 2, 64, 64), (40, 1, 32, 16)])
@pytest.mark.parametrize("splits", [None, 1, 7])
def test_attention_bf16_decode(nq, nkv, d, page, splits, monkeypatch):
    rows = [(700, 1), (0, 1), (15, 1), (16, 1), (63, 1), (64, 1), (333, 1)]
    pb, q, ref, scale = _attention_case(torch.bfloat16, rows, nq, nkv, d, page, needle=3)
    if splits is not None:
        monkeypatch.setattr(attention_bf16, "choose_splits", lambda *a, **k: splits)
    out = torch.full_like(q, float("nan"))
    ctx = make_context(pb)
    assert ctx.decode_only
    attention_bf16.run(out, q, pb.k_pool, pb.v_pool, ctx, 0, scale, None)
    assert ref[0, 0].mean().item() > 40  # the far key dominates row 0
    assert torch.allclose(out.float(), ref, atol=0.3, rtol=2e-2)
    assert torch.allclose(out.float()[1:3], ref[1:3], **BF16_TOL)


@pytest.mark.parametrize("graph_kv_len", [0, 8192, 32768])
def test_attention_bf16_decode_of_long_contexts_as_laid_out_inside_a_graph(graph_kv_len):
    """Inside a CUDA graph the launch follows the batch size and the graph's class of context length, not
    the rows' lengths: a short class cuts the keys 8 ways as one cluster, the long classes as many ways as
    CTAs fit the GPU (merged through scratch memory by the last CTA to finish). Rows far shorter than the
    class leave most of their splits without keys. One key far back carries row 0's result."""
    seen = []
    choose = attention_bf16.choose_splits

    def spy(*a, **k):
        seen.append(choose(*a, **k))
        return seen[-1]

    import unittest.mock as mock

    rows = [(9000, 1), (40, 1), (8191, 1)]
    pb, q, ref, scale = _attention_case(torch.bfloat16, rows, 4, 2, 128, 16, needle=3)
    ctx = make_context(pb)
    ctx.graph_bucket, ctx.graph_kv_len = 4, graph_kv_len
    out = torch.full_like(q, float("nan"))
    with mock.patch.object(attention_bf16, "choose_splits", spy):
        attention_bf16.run(out, q, pb.k_pool, pb.v_pool, ctx, 0, scale, None)
    assert seen == [{0: 8, 8192: 32, 32768: 49}[graph_kv_len]]  # 3 rows x 2 head groups share 296 CTAs
    assert ref[0, 0].mean().item() > 40  # the far key dominates row 0
    assert torch.allclose(out.float(), ref, atol=0.3, rtol=2e-2)
    assert torch.allclose(out.float()[1:2], ref[1:2], **BF16_TOL)


def test_the_device_says_how_many_clusters_of_decode_ctas_it_holds():
    """Key splits that run as a cluster are chosen so that every cluster is resident at once; the number
    comes from the device (a cluster lies within one GPC, so it is less than SMs x CTAs per SM / size)."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    counts = [attention_bf16.clusters_resident(128, n) for n in range(1, 9)]
    assert all(c >= 1 for c in counts) and counts == sorted(counts, reverse=True)
    assert counts[0] <= 4 * sms and all(n * c <= counts[0] for n, c in zip(range(1, 9), counts))
    splits = attention_bf16.choose_splits(8, 8, None, sms, lambda n: attention_bf16.clusters_resident(128, n))
    assert 1 <= splits <= 8 and (splits == 1 or attention_bf16.clusters_resident(128, splits) >= 64)


@pytest.mark.parametrize("window", [1, 16, 17, 100])
def test_attention_bf16_decode_window_edge(window):
    rows = [(200, 1), (5, 1), (99, 1), (100, 1)]
    pb, q, ref, scale = _attention_case(torch.bfloat16, rows, 6, 2, 48, 8, window=window)
    out = torch.full_like(q, float("nan"))
    attention_bf16.run(out, q, pb.k_pool, pb.v_pool, make_context(pb), 0, scale, window)
    assert torch.allclose(out.float(), ref, **BF16_TOL)


@pytest.fixture(params=[None, (2, 1), (3, 2), (8, 1)], ids=lambda p: "auto" if p is None else f"splits{p[0]}x{p[1]}")
def key_splits(request, monkeypatch):
    """Forces how the tcgen05 attention cuts a tile's keys between CTAs (None: its own choice, which
    is no cut for steps as small as a test's): (splits, least key tiles per split)."""
    monkeypatch.setattr(ops, "ATTN_TC_SPLITS", request.param)
    return request.param


TC_SHAPES = [(16, 8, 128, 16), (8, 8, 128, 8), (32, 8, 128, 32), (8, 1, 128, 16), (4, 2, 128, 128), (6, 2, 128, 64)]


@pytest.mark.parametrize("nq, nkv, d, page", TC_SHAPES)
def test_attention_tcgen05_prompts_and_mixed_steps(nq, nkv, d, page, key_splits):
    rows = [(0, 37), (52, 1), (15, 18), (0, 1), (63, 2), (0, 150), (100, 70), (64, 64), (0, 300), (250, 130), (0, 700), (900, 260)]
    pb, q, ref, scale = _attention_case(torch.bfloat16, rows, nq, nkv, d, page)
    assert ops.attention_tc_ok(q, pb.k_pool)
    out = torch.full_like(q, float("nan"))
    ops.attention_tc_prefill(out, q, pb.k_pool, pb.v_pool, make_context(pb), 0, scale, None)
    torch.cuda.synchronize()
    assert ops.device_status("cuda").item() == 0
    assert torch.allclose(out.float(), ref, **BF16_TOL)


@pytest.mark.parametrize("window", [1, 7, 128, 129, 200])
def test_attention_tcgen05_window_edge(window, key_splits):
    rows = [(0, 400), (130, 3), (399, 1), (256, 128)]
    pb, q, ref, scale = _attention_case(torch.bfloat16, rows, 4, 2, 128, 16, window=window)
    out = torch.full_like(q, float("nan"))
    ops.attention_tc_prefill(out, q, pb.k_pool, pb.v_pool, make_context(pb), 0, scale, window)
    torch.cuda.synchronize()
    assert ops.device_status("cuda").item() == 0
    assert torch.allclose(out.float(), ref, **BF16_TOL)


def test_attention_tcgen05_finds_a_far_key_and_survives_poisoned_pages(key_splits):
    rows = [(0, 700), (900, 5)]
    pb, q, ref, scale = _attention_case(torch.bfloat16, rows, 4, 2, 128, 16, needle=3)
    out = torch.full_like(q, float("nan"))  # pages past each request's end are NaN (PagedBatch poisons them)
    ops.attention_tc_prefill(out, q, pb.k_pool, pb.v_pool, make_context(pb), 0, scale, None)
    torch.cuda.synchronize()
    assert ops.device_status("cuda").item() == 0
    assert ref[699, 0].mean().item() > 40 and ref[-1, 0].mean().item() > 40
    assert torch.allclose(out.float(), ref, atol=0.3, rtol=2e-2)


def test_attention_tcgen05_large_scores_keep_the_lazy_rescale_exact(key_splits):
    """Scores that keep growing along the keys force the running maximum up tile after tile."""
    torch.manual_seed(3)
    nq, nkv, d, page, n = 2, 1, 128, 16, 600
    pb = PagedBatch([(0, n)], page, nkv, d, torch.bfloat16, seed=1)
    k = torch.randn(n, nkv, d, device=DEV)
    k[:, 0, 0] = torch.linspace(0, 40, n, device=DEV)  # a component that grows with the position
    v = torch.randn(n, nkv, d, device=DEV)
    q = torch.randn(n, nq, d, device=DEV) * 0.1
    q[:, :, 0] = 11.0
    k, v, q = k.bfloat16(), v.bfloat16(), q.bfloat16()
    pb.fill(0, k, v)
    ref = reference_attention(q, k, v, list(range(n)), d ** -0.5)
    out = torch.full_like(q, float("nan"))
    ops.attention_tc_prefill(out, q, pb.k_pool, pb.v_pool, make_context(pb), 0, d ** -0.5, None)
    torch.cuda.synchronize()
    assert ops.device_status("cuda").item() == 0
    assert torch.allclose(out.float(), ref, **BF16_TOL)


@pytest.mark.parametrize("nq, nkv, d, page", [(16, 8, 128, 16), (8, 2, 64, 16), (6, 2, 48, 8)])
@pytest.mark.parametrize("window", [None, 33])
def test_attention_of_a_mixed_step_uses_both_kernels(nq, nkv, d, page, window):
    """Decoding requests come first in a mixed step: they go to the split-key kernel, the prompt
    portions behind them (and a single token that follows a portion) to the tiled kernel."""
    from miniserve_b200.ops import native

    rows = [(700, 1), (15, 1), (0, 1), (0, 37), (100, 70), (52, 1), (0, 300)]
    pb, q, ref, scale = _attention_case(torch.bfloat16, rows, nq, nkv, d, page, window=window, needle=3)
    ctx = make_context(pb)
    assert ctx.leading_single_rows == 3 and not ctx.decode_only
    out = torch.full_like(q, float("nan"))
    before = native.LAUNCHES[0]
    ops.attention(out, q, pb.k_pool, pb.v_pool, ctx, 0, scale, window)
    assert native.LAUNCHES[0] - before == 2
    torch.cuda.synchronize()
    assert ops.device_status("cuda").item() == 0
    assert torch.allclose(out.float()[1:], ref[1:], **BF16_TOL)
    assert torch.allclose(out.float()[:1], ref[:1], atol=0.3, rtol=2e-2)  # the far key's value is 50


def test_attention_bf16_refuses_other_head_sizes():
    assert not attention_bf16.supports(40, 16) and not attention_bf16.supports(272, 16)
    with pytest.raises(ValueError):
        attention_bf16._lib(40)


# ------------------------------------------------------------------ sampling
@pytest.mark.parametrize("vocab", [5, 503, 151936])
def test_argmax_first_index_wins(vocab):
    logits = torch.randn(7, vocab, device=DEV)
    logits[2, 3] = logits[2, vocab - 1] = 99.0  # a tie: the lower index wins
    logits[4, :] = 1.0
    tokens = torch.empty(7, dtype=torch.int32, device=DEV)
    ops.sample(tokens, logits)
    expect = torch.argmax(logits, -1)
    assert tokens.tolist() == expect.tolist() and tokens[2].item() == 3 and tokens[4].item() == 0


def _sample(logits, temps, top_ps, seeds, counters):
    rows = logits.shape[0]
    tokens = torch.empty(rows, dtype=torch.int32, device=DEV)
    scratch = torch.empty(rows * ops.nucleus_bytes(), dtype=torch.uint8, device=DEV)
    use_p = top_ps is not None
    ops.sample(tokens, logits, temperature=torch.tensor(temps, device=DEV),
               top_p=torch.tensor(top_ps, device=DEV) if use_p else None,
               seed=torch.tensor(seeds, dtype=torch.int64, device=DEV),
               counter=torch.tensor(counters, dtype=torch.int64, device=DEV), scratch=scratch if use_p else None)
    return tokens.tolist()


def test_temperature_sampling_matches_the_plain_sampler_and_ignores_neighbours():
    vocab = 503
    logits = torch.randn(6, vocab, device=DEV) * 2
    temps = [0.7, 0.0, 1.3, 0.7, 1.0, 0.0]
    seeds = [1, 2, 4000000000, 1, 77, 5]
    counters = [10, 11, 12, 10, 300, 1]
    got = _sample(logits, temps, None, seeds, counters)
    for r in range(6):
        assert got[r] == plain.sample_token(logits[r].cpu(), temps[r], seeds[r], counters[r])
    # the same (seed, counter, logits) samples the same token anywhere in any batch
    alone = _sample(logits[3:4].contiguous(), [0.7], None, [1], [10])
    assert alone[0] == got[3]
    assert _sample(logits, temps, None, seeds, [c + 1 for c in counters]) != got


def test_top_p_matches_the_plain_sampler():
    vocab = 300
    torch.manual_seed(1)
    logits = torch.randn(40, vocab, device=DEV) * 3
    logits[5, :] = 0.0           # all ties: the nucleus keeps the first tokens in index order
    logits[6, 10:20] = 7.0       # a tied group at the cut
    temps = [1.0] * 40
    tops = [0.05 + 0.9 * (i % 10) / 10 for i in range(40)]
    tops[7] = 1.0
    seeds = list(range(100, 140))
    counters = list(range(40))
    got = _sample(logits, temps, tops, seeds, counters)
    same = sum(got[r] == plain.sample_token(logits[r].cpu(), temps[r], seeds[r], counters[r], tops[r]) for r in range(40))
    assert same >= 39  # a cut that falls within rounding of top_p may go either way
    # every sampled token lies inside its row's nucleus
    for r in range(40):
        p = torch.softmax(logits[r].cpu().float(), -1)
        sp, order = torch.sort(p, descending=True, stable=True)
        keep = (torch.cumsum(sp, 0) - sp) < tops[r] + 1e-6
        assert got[r] in set(order[keep].tolist())
    assert got[5] < max(1, int(0.55 * vocab) + 2)


@pytest.mark.parametrize("vocab", [20011, 151936, 420000])
def test_top_p_over_a_large_vocabulary_matches_the_plain_sampler(vocab):
    """From 16,384 tokens on a row's nucleus is found by a thread-block cluster of 8 CTAs that keep the row's
    probabilities in shared memory; beyond what that holds (420,000 here) by one CTA that walks the row."""
    torch.manual_seed(vocab)
    rows = 9
    logits = torch.randn(rows, vocab, device=DEV) * 4
    logits[1, :] = 0.5                      # all ties: the first tokens in index order are kept
    logits[2, 1000:1040] = 9.0              # a tied group at the cut, across a warp's and (at 151,936) no CTA's edge
    logits[2, vocab - 3:] = 9.0             # ... and in the last CTA's stretch
    logits[3, 7] = 30.0                     # one token holds nearly all the mass
    temps = [0.9, 1.0, 1.0, 1.0, 0.0, 0.8, 1.3, 0.6, 1.0]
    tops = [0.9, 0.3, 0.35, 0.5, 0.9, 1.0, 0.99, 0.05, 0.7]
    seeds = list(range(50, 50 + rows))
    counters = list(range(3, 3 + rows))
    got = _sample(logits, temps, tops, seeds, counters)
    expect = [plain.sample_token(logits[r].cpu(), temps[r], seeds[r], counters[r], tops[r]) for r in range(rows)]
    same = sum(g == e for g, e in zip(got, expect))
    assert same >= rows - 1, (got, expect)  # a cut that falls within rounding of top_p may go either way
    for r in range(rows):
        if temps[r] == 0 or tops[r] >= 1:
            assert got[r] == expect[r]
            continue
        p = torch.softmax(logits[r].cpu().float() / temps[r], -1)
        sp, order = torch.sort(p, descending=True, stable=True)
        keep = (torch.cumsum(sp, 0) - sp) < tops[r] + 1e-5
        assert got[r] in set(order[keep].tolist()), r
    assert got[1] < int(0.3 * vocab) + 2 and got[3] == 7
    # the same rows alone and in another order give the same tokens
    perm = [4, 8, 0, 2]
    again = _sample(logits[perm].contiguous(), [temps[i] for i in perm], [tops[i] for i in perm], [seeds[i] for i in perm],
                    [counters[i] for i in perm])
    assert again == [got[i] for i in perm]


def test_top_p_distribution():
    vocab = 8
    probs = torch.tensor([0.4, 0.25, 0.15, 0.1, 0.05, 0.03, 0.01, 0.01])
    rows = 20000
    logits = probs.log().repeat(rows, 1).to(DEV).contiguous()
    got = torch.tensor(_sample(logits, [1.0] * rows, [0.7] * rows, list(range(rows)), [3] * rows))
    freq = torch.bincount(got, minlength=vocab).float() / rows
    expect = torch.tensor([0.4, 0.25, 0.15, 0, 0, 0, 0, 0]) / 0.8
    assert (freq - expect).abs().max().item() < 0.015


def test_a_wait_that_nothing_answers_gives_up_raises_the_status_word_and_leaves_the_device_usable():
    """The tensor-core pipelines wait on mbarriers with a time limit and raise the device status word when
    it runs out. Here a kernel waits on a barrier that nobody arrives on, with a limit of 50 ms: it ends
    by itself, the word says so, and the next kernel runs."""
    import time

    from miniserve_b200.ops import native

    k = native.kernels()
    word = torch.zeros(1, dtype=torch.int32, device=DEV)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    native.kernel_check(k.ms_wait_selftest(word.data_ptr(), 50_000_000, 77, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    took = time.perf_counter() - t0
    assert word.item() == 77
    assert 0.04 <= took < 1.0, f"the wait of 50 ms took {took:.3f} s"
    out = torch.empty(5, 24, device=DEV)
    table = torch.randn(7, 24, device=DEV)
    ids = torch.arange(5, device=DEV, dtype=torch.int32)
    ops.embed_gather(out, table, ids)
    assert torch.equal(out, table[:5])
