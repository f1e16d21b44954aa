"""The decode-attention entry point that allocates nothing (csrc/attention_noalloc.h).

It is for embedders that must not call cudaMalloc or any allocating library routine while they
run the kernels (a real-time loop, a plugin that may not own memory, a process whose memory
budget is fixed): the split-K scratch lives in a device array inside the library. The test calls
it through its exported C symbol, twice in a row, and compares it with the ordinary entry point,
whose scratch the caller allocates. This file is collected last on purpose: a run that stops at
the first failure has then already run every other test.
"""

import ctypes

import pytest
import torch

from miniserve_b200.ops import attention_bf16
from tests.kernel_util import PagedBatch, reference_attention

pytestmark = pytest.mark.gpu

SCRATCH_FLOATS = 1 << 20


def _symbol(d):
    fns = attention_bf16._lib(d)
    fn = getattr(fns["lib"], f"ms_attn_bf16_d{d}_decode_noalloc")
    p, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [p, p, p, p, p, p, p, i, i, i, f, i, i, i, p]
    fn.restype = ctypes.c_int
    return fns, fn


@pytest.mark.parametrize("nq, nkv, d, page, splits", [(16, 8, 128, 16, 4), (6, 1, 32, 8, 3), (4, 2, 64, 16, 1)])
def test_decode_without_allocation_matches_the_allocating_entry_point(nq, nkv, d, page, splits):
    torch.manual_seed(0)
    rows = [(300, 1), (17, 1), (64, 1), (1000, 1), (0, 1)]
    pb = PagedBatch(rows, page, nkv, d, torch.bfloat16, seed=2)
    scale = d ** -0.5
    qs, refs = [], []
    for r, (s, n) in enumerate(rows):
        k = torch.randn(s + n, nkv, d, device="cuda").bfloat16()
        v = torch.randn(s + n, nkv, d, device="cuda").bfloat16()
        q = torch.randn(n, nq, d, device="cuda").bfloat16()
        pb.fill(r, k, v)
        qs.append(q)
        refs.append(reference_attention(q, k, v, [s], scale))
    q, ref = torch.cat(qs).contiguous(), torch.cat(refs)
    fns, noalloc = _symbol(d)
    stream = torch.cuda.current_stream().cuda_stream

    # the ordinary entry point, scratch allocated by the caller
    items = len(rows) * nq * splits
    part_o = torch.empty(items * d, dtype=torch.float32, device="cuda")
    part_ml = torch.empty(items * 2, dtype=torch.float32, device="cuda")
    expect = torch.full_like(q, float("nan"))
    rc = fns["decode"](expect.data_ptr(), part_o.data_ptr(), part_ml.data_ptr(), q.data_ptr(), pb.k_pool.data_ptr(),
                       pb.v_pool.data_ptr(), pb.kv_len.data_ptr(), pb.page_indptr.data_ptr(), pb.page_indices.data_ptr(),
                       len(rows), nq, nkv, scale, 0, page, splits, stream)
    assert rc == 0
    assert torch.allclose(expect.float(), ref, atol=2e-2, rtol=2e-2)

    # the entry point that allocates nothing: two calls in a row share the built-in scratch
    outs = []
    for attempt in range(2):
        out = torch.full_like(q, float("nan"))
        torch.cuda.synchronize()
        # what the device itself says is free: a cudaMalloc inside the library would show here, which the
        # tensor library's own counters would not see
        before = torch.cuda.mem_get_info()[0]
        rc = noalloc(out.data_ptr(), q.data_ptr(), pb.k_pool.data_ptr(), pb.v_pool.data_ptr(), pb.kv_len.data_ptr(),
                     pb.page_indptr.data_ptr(), pb.page_indices.data_ptr(), len(rows), nq, nkv, scale, 0, page, splits,
                     stream)
        assert rc == 0, fns["last_error"]().decode()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == before
        outs.append(out)
    for out in outs:
        assert torch.allclose(out.float(), expect.float(), atol=2e-2, rtol=2e-2)
        assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2)
    assert torch.equal(outs[0], outs[1])


def test_decode_without_allocation_refuses_what_does_not_fit():
    d, nq, nkv, page = 128, 16, 8, 16
    fns, noalloc = _symbol(d)
    rows, splits = 64, 8  # 64 * 16 * 8 * 130 floats > 2**20
    assert rows * nq * splits * (d + 2) > SCRATCH_FLOATS
    dummy = torch.zeros(8, dtype=torch.int32, device="cuda")
    rc = noalloc(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                 dummy.data_ptr(), dummy.data_ptr(), rows, nq, nkv, 0.1, 0, page, splits,
                 torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    msg = fns["last_error"]().decode()
    assert "scratch" in msg and str(SCRATCH_FLOATS) in msg
    torch.cuda.synchronize()
