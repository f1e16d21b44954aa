"""The persistent decode-chain kernel (``csrc/decode_chain.cu``) and the decode attention that takes
the q|k|v projection as it is, each against plain PyTorch float32 arithmetic and against the
separate kernels they replace, at sizes other than the engine's."""

import pytest
import torch

from miniserve_b200 import ops
from miniserve_b200.ops import attention_bf16
from miniserve_b200.ops import decode_chain as chain
from tests.kernel_util import PagedBatch, make_context, reference_attention
from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


def _sync_state():
    return torch.zeros(4, dtype=torch.int32, device=DEV)


def _bf(x):
    return x.to(BF).float()


def _run(phases, rows, sync=None, persistent=True):
    sync = sync if sync is not None else _sync_state()
    status = ops.device_status(DEV)
    chain.run(phases, rows, sync, status, torch.cuda.current_stream().cuda_stream, persistent=persistent)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert sync[2].item() == 0  # nobody gave up


@pytest.mark.parametrize("m", [1, 5, 8, 9, 16])
@pytest.mark.parametrize("n, k", [(4096, 1024), (1024, 2048), (503, 96), (72, 3072), (20000, 264), (1024, 4104)])
@pytest.mark.parametrize("out_f32", [False, True])
@pytest.mark.parametrize("persistent", [True, False], ids=["one_kernel", "kernel_per_phase"])
def test_chain_single_product_with_the_row_scale_of_a_norm(m, n, k, out_f32, persistent):
    torch.manual_seed(m + n + k)
    x = torch.randn(m, k, device=DEV).to(BF)
    w = (torch.randn(n, k, device=DEV) * k ** -0.5).to(BF)
    parts = 7
    sumsq = torch.rand(m, parts, device=DEV) * k
    eps = 1e-5
    scale = torch.rsqrt(sumsq.sum(-1, keepdim=True) / k + eps)
    expect = (x.float() @ w.float().T) * scale
    out = torch.full((m, n), float("nan"), device=DEV, dtype=torch.float32 if out_f32 else BF)
    _run([chain.Phase(w, x, chain.OUT_F32 if out_f32 else chain.OUT_BF16, out=out, sumsq_in=sumsq, eps=eps)], m, persistent=persistent)
    tol = dict(atol=2e-3, rtol=2e-3) if out_f32 else dict(atol=3e-2, rtol=2e-2)
    assert torch.allclose(out.float(), expect, **tol)
    # a row's result does not depend on the rows beside it
    if m > 1:
        alone = torch.empty((1, n), device=DEV, dtype=out.dtype)
        _run([chain.Phase(w, x[m - 1:].contiguous(), chain.OUT_F32 if out_f32 else chain.OUT_BF16, out=alone,
                          sumsq_in=sumsq[m - 1:].contiguous(), eps=eps)], 1, persistent=not persistent)
        assert torch.equal(alone[0], out[m - 1])  # nor on which of the two forms ran


def _layer_reference(res, mixed, w_o, nw2, eps2, w_gu, w_down, nw_next, eps_next, w_next):
    """float32 arithmetic with the chain's rounding points."""
    inter = w_down.shape[1]
    r1 = res + _bf(mixed.float() @ w_o.float().T)
    xw1 = _bf(r1 * nw2.float())
    s1 = torch.rsqrt((r1 * r1).sum(-1, keepdim=True) / r1.shape[1] + eps2)
    gu = xw1 @ w_gu.float().T
    g, u = _bf(gu[:, :inter] * s1), _bf(gu[:, inter:] * s1)
    act = _bf(g * torch.sigmoid(g) * u)
    r2 = r1 + _bf(act @ w_down.float().T)
    xw2 = _bf(r2 * nw_next.float())
    s2 = torch.rsqrt((r2 * r2).sum(-1, keepdim=True) / r2.shape[1] + eps_next)
    return r2, (xw2 @ w_next.float().T) * s2


@pytest.mark.parametrize("m", [1, 3, 8, 13, 16])
@pytest.mark.parametrize("hidden, mixed_w, inter, n_next", [(1024, 2048, 3072, 4096), (96, 192, 224, 256), (64, 64, 128, 130),
                                                            (200, 104, 72, 1000)])
def test_chain_of_a_layer_tail_and_the_next_projection(m, hidden, mixed_w, inter, n_next):
    """o -> +residual, norm -> gate|up, SiLU * up -> down -> +residual, norm -> next projection, one launch."""
    torch.manual_seed(m + hidden)
    res = torch.randn(m, hidden, device=DEV) * 2
    mixed = torch.randn(m, mixed_w, device=DEV).to(BF)
    w_o = (torch.randn(hidden, mixed_w, device=DEV) * mixed_w ** -0.5).to(BF)
    w_gu = (torch.randn(2 * inter, hidden, device=DEV) * hidden ** -0.5).to(BF)
    w_down = (torch.randn(hidden, inter, device=DEV) * inter ** -0.5).to(BF)
    w_next = (torch.randn(n_next, hidden, device=DEV) * hidden ** -0.5).to(BF)
    nw2 = (1 + 0.1 * torch.randn(hidden, device=DEV)).to(BF)
    nw3 = (1 + 0.1 * torch.randn(hidden, device=DEV)).to(BF)
    eps2, eps3 = 1e-6, 1e-5
    want_res, want_out = _layer_reference(res, mixed, w_o, nw2, eps2, w_gu, w_down, nw3, eps3, w_next)

    parts = chain.tiles(hidden)
    residual = res.clone()
    xw_a, xw_b = (torch.empty(m, hidden, device=DEV, dtype=BF) for _ in range(2))
    ss_a, ss_b = (torch.full((m, parts), float("nan"), device=DEV) for _ in range(2))
    act = torch.empty(m, inter, device=DEV, dtype=BF)
    out = torch.full((m, n_next), float("nan"), device=DEV, dtype=BF)
    phases = [
        chain.Phase(w_o, mixed, chain.RESIDUAL, residual=residual, norm_w=nw2, xw_out=xw_b, sumsq_out=ss_b),
        chain.Phase(w_gu, xw_b, chain.SILU_MUL, out=act, sumsq_in=ss_b, eps=eps2),
        chain.Phase(w_down, act, chain.RESIDUAL, residual=residual, norm_w=nw3, xw_out=xw_a, sumsq_out=ss_a),
        chain.Phase(w_next, xw_a, chain.OUT_BF16, out=out, sumsq_in=ss_a, eps=eps3),
    ]
    sync = _sync_state()
    _run(phases, m, sync)
    assert torch.allclose(residual, want_res, atol=3e-2, rtol=1e-2)
    assert torch.allclose(ss_a.sum(-1), (residual * residual).sum(-1), rtol=1e-4)
    assert torch.allclose(out.float(), want_out, atol=6e-2, rtol=3e-2)
    # the separate kernels the chain replaces give the same function (they round at other places)
    r = res.clone()
    x1 = torch.empty(m, hidden, device=DEV, dtype=BF)
    ops.add_rmsnorm(x1, r, ops.linear(mixed, w_o), nw2, eps2)
    a = torch.empty(m, inter, device=DEV, dtype=BF)
    ops.linear_silu_mul(x1, w_gu, a)
    x2 = torch.empty(m, hidden, device=DEV, dtype=BF)
    ops.add_rmsnorm(x2, r, ops.linear(a, w_down), nw3, eps3)
    sep = ops.linear(x2, w_next)
    assert torch.allclose(out.float(), sep.float(), atol=8e-2, rtol=4e-2)
    # run again on the same barrier state (it is left ready), as one kernel per phase, and with a row
    # alone: the same bits
    for persistent in (True, False):
        residual2, out2 = res.clone(), torch.empty_like(out)
        phases[0].residual = phases[2].residual = residual2
        phases[3].out = out2
        _run(phases, m, sync, persistent=persistent)
        assert torch.equal(out2, out) and torch.equal(residual2, residual)
    if m > 1:
        residual1, out1 = res[m - 1:].clone(), torch.empty((1, n_next), device=DEV, dtype=BF)
        phases[0].x = mixed[m - 1:].contiguous()
        phases[0].residual = phases[2].residual = residual1
        phases[3].out = out1
        _run(phases, 1, sync)
        assert torch.equal(out1[0], out[m - 1])


def test_chain_embed_prepares_the_first_norm():
    vocab, hidden, t = 333, 200, 7
    table = torch.randn(vocab, hidden, device=DEV).to(BF)
    nw = (1 + 0.1 * torch.randn(hidden, device=DEV)).to(BF)
    ids = torch.randint(0, vocab, (t,), device=DEV, dtype=torch.int32)
    ids[0], ids[-1] = vocab - 1, 0
    residual = torch.empty(t, hidden, device=DEV)
    xw = torch.empty(t, hidden, device=DEV, dtype=BF)
    ss = torch.empty(t, 1, device=DEV)
    chain.embed(residual, xw, ss, table, ids, nw, torch.cuda.current_stream().cuda_stream)
    want = table[ids.long()].float()
    assert torch.equal(residual, want)
    assert torch.equal(xw, (want * nw.float()).to(BF))
    assert torch.allclose(ss[:, 0], (want * want).sum(-1), rtol=1e-5)


def test_chain_refuses_what_it_cannot_run():
    x = torch.zeros(2, 16, device=DEV, dtype=BF)
    w = torch.zeros(8, 16, device=DEV, dtype=BF)
    out = torch.zeros(2, 8, device=DEV, dtype=BF)
    assert not chain.fits(8, 20000)  # the activations alone would not fit a CTA's shared memory
    assert chain.fits(16, 3072) and not chain.fits(17, 64)
    with pytest.raises(ops.NativeError, match="multiple of 8"):
        bad = torch.zeros(8, 12, device=DEV, dtype=BF)
        chain.run([chain.Phase(bad, torch.zeros(2, 12, device=DEV, dtype=BF), chain.OUT_BF16, out=out)], 2, _sync_state(),
                  ops.device_status(DEV), torch.cuda.current_stream().cuda_stream)
    with pytest.raises(AssertionError):
        chain.run([chain.Phase(w, x, chain.OUT_BF16, out=out)] * 9, 2, _sync_state(), ops.device_status(DEV), 0)


@pytest.mark.parametrize("nq, nkv, d, page", [(16, 8, 128, 16), (4, 2, 16, 16), (6, 1, 32, 8), (8, 8, 48, 4), (5, 5, 80, 32),
                                              (2, 1, 256, 16), (40, 1, 32, 16), (8, 2, 64, 64)])
@pytest.mark.parametrize("splits", [None, 1, 3, 11])
@pytest.mark.parametrize("rotate, normed, window", [(True, True, None), (False, True, 33), (True, False, None), ("half", True, None)])
def test_decode_attention_takes_the_projection_as_it_is(nq, nkv, d, page, splits, rotate, normed, window, monkeypatch):
    """The decode kernel that norms and rotates q and k itself and writes the cache, against the
    separate kernel followed by the decode kernel, and against float32 attention."""
    torch.manual_seed(nq * d + page)
    rows = [(700, 1), (0, 1), (15, 1), (16, 1), (63, 1), (64, 1), (333, 1)]
    pb = PagedBatch(rows, page, nkv, d, BF, seed=nq)
    t = len(rows)
    theta, eps, scale = 1e6, 1e-6, d ** -0.5
    rot = 0 if not rotate else (d // 2 if rotate == "half" else d)
    old = []
    for r, (s, _) in enumerate(rows):
        k = torch.randn(s + 1, nkv, d, device=DEV).to(BF)
        v = torch.randn(s + 1, nkv, d, device=DEV).to(BF)
        pb.fill(r, k, v, upto=s)  # the newest position keeps the pool's NaN until a kernel writes it
        old.append((k, v))
    qkv = (torch.randn(t, (nq + 2 * nkv) * d, device=DEV) * 1.5).to(BF)
    qw = (1 + 0.2 * torch.randn(d, device=DEV)).to(BF) if normed else None
    kw = (1 + 0.2 * torch.randn(d, device=DEV)).to(BF) if normed else None
    inv_freq = (1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.int64).float() / rot))).to(DEV) if rot else None
    table = ops.rope_table(pb.positions, inv_freq, t, rot) if rot else None
    if splits is not None:
        monkeypatch.setattr(attention_bf16, "choose_splits", lambda *a, **k: splits)
    # the separate kernels
    k1, v1 = pb.k_pool.clone(), pb.v_pool.clone()
    q1 = torch.empty(t, nq, d, device=DEV, dtype=BF)
    ops.qk_norm_rope_kv(q1, k1, v1, qkv, qw, kw, inv_freq, rot, eps, pb.positions, pb.row_of_token, pb.page_indptr,
                        pb.page_indices, page, pb.status, cos_sin=table)
    out1 = torch.full((t, nq, d), float("nan"), device=DEV, dtype=BF)
    ctx = make_context(pb)
    attention_bf16.run_decode(out1, q1, k1, v1, ctx, 0, scale, window, t)
    # the one kernel
    k2, v2 = pb.k_pool.clone(), pb.v_pool.clone()
    out2 = torch.full((t, nq, d), float("nan"), device=DEV, dtype=BF)
    attention_bf16.run_decode(out2, None, k2, v2, ctx, 0, scale, window, t,
                              projection=dict(qkv=qkv, q_norm_w=qw, k_norm_w=kw, cos_sin=table, rot=rot, eps=eps))
    torch.cuda.synchronize()
    assert pb.status.item() == 0
    for r, (s, _) in enumerate(rows):  # the new key and value are in the cache, where the separate kernel puts them
        got_k, got_v = pb.read(r, k2, s + 1)[s], pb.read(r, v2, s + 1)[s]
        ref_k, ref_v = pb.read(r, k1, s + 1)[s], pb.read(r, v1, s + 1)[s]
        assert torch.equal(got_v, ref_v)
        assert torch.allclose(got_k.float(), ref_k.float(), atol=2e-2, rtol=2e-2)
    assert torch.allclose(out2.float(), out1.float(), atol=3e-2, rtol=3e-2)
    assert torch.equal(torch.isnan(k2), torch.isnan(k1))  # nothing else was written
    # against float32 attention over the keys as the separate kernel stored them
    for r, (s, _) in enumerate(rows):
        kk, vv = pb.read(r, k1, s + 1), pb.read(r, v1, s + 1)
        ref = reference_attention(q1[r:r + 1], kk, vv, [s], scale, window)
        assert torch.allclose(out2[r:r + 1].float(), ref, atol=3e-2, rtol=3e-2)


def test_decode_attention_from_the_projection_reports_a_missing_page():
    rows = [(40, 1)]
    pb = PagedBatch(rows, 8, 1, 32, BF)
    pb.page_indices[40 // 8] = -1  # the newest position's page was given back
    k = torch.randn(41, 1, 32, device=DEV).to(BF)
    pb.fill(0, k, k, upto=40)
    qkv = torch.randn(1, 3 * 32, device=DEV).to(BF)
    out = torch.empty(1, 1, 32, device=DEV, dtype=BF)
    attention_bf16.run_decode(out, None, pb.k_pool, pb.v_pool, make_context(pb), 0, 0.2, None, 1,
                              projection=dict(qkv=qkv, q_norm_w=None, k_norm_w=None, cos_sin=None, rot=0, eps=0.0))
    torch.cuda.synchronize()
    assert pb.status.item() == 2
    pb.status.zero_()
