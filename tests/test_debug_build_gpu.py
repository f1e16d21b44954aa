"""The debug build of the kernels (MINISERVE_DEBUG=1: -DMS_DEBUG_CHECKS, libraries under names of
their own): a page id beyond the pool raises the status word and the access is skipped. The id used
here lies beyond the page count the kernel is TOLD but inside the memory that is really there, so
the test is harmless even for a build without the check."""

import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

SCRIPT = textwrap.dedent("""
    import torch
    from miniserve_b200 import ops
    from miniserve_b200.ops import build, native
    assert build.debug_checks()
    dev = "cuda"
    pages, told, nkv, page, d, nq = 12, 8, 2, 8, 32, 4
    k_pool = torch.full((pages, nkv, page, d), float("nan"), device=dev)
    v_pool = torch.full_like(k_pool, float("nan"))
    i32 = dict(dtype=torch.int32, device=dev)
    positions, row_of = torch.tensor([3, 9], **i32), torch.tensor([0, 1], **i32)
    indptr = torch.tensor([0, 1, 3], **i32)
    status = torch.zeros(1, **i32)
    qkv = torch.randn(2, (nq + 2 * nkv) * d, device=dev)
    q_out = torch.empty(2, nq, d, device=dev)
    k = native.kernels()

    def write(indices):
        native.kernel_check(k.ms_qk_norm_rope_kv(
            q_out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), qkv.data_ptr(), None, None, None, None, positions.data_ptr(),
            row_of.data_ptr(), indptr.data_ptr(), indices.data_ptr(), 2, nq, nkv, d, 0, 1e-6, page, told, status.data_ptr(), 0,
            torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()

    write(torch.tensor([1, 2, 10], **i32))       # token 1 (position 9) lives in page 10: beyond the 8 the kernel was told
    assert status.item() == 5, status.item()
    assert torch.isnan(k_pool[10]).all()         # the write was skipped
    assert not torch.isnan(k_pool[1, :, 3]).any()  # token 0 was written
    status.zero_()
    write(torch.tensor([1, 2, 5], **i32))
    assert status.item() == 0 and not torch.isnan(k_pool[5, :, 1]).any()

    # the reader: row-wise attention over the same tables
    q = torch.randn(2, nq, d, device=dev)
    out = torch.empty_like(q)
    k_pool.nan_to_num_(0.0); v_pool.nan_to_num_(0.0)

    def read(indices):
        native.kernel_check(k.ms_attention_rowwise(
            out.data_ptr(), q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), positions.data_ptr(), row_of.data_ptr(),
            indptr.data_ptr(), indices.data_ptr(), 2, nq, nkv, d, 0.2, 0, page, told, status.data_ptr(), 0,
            torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()

    read(torch.tensor([1, 2, 11], **i32))
    assert status.item() == 5, status.item()
    status.zero_()
    read(torch.tensor([1, 2, 5], **i32))
    assert status.item() == 0
    print("debug build ok", Path(build.ensure_built(build.KERNELS)).name)
""")


def test_debug_build_raises_the_status_word_for_a_page_id_beyond_the_pool(tmp_path):
    root = Path(__file__).resolve().parent.parent
    env = dict(os.environ, MINISERVE_DEBUG="1", MINISERVE_BUILD_DIR=str(tmp_path), PYTHONPATH=str(root))
    proc = subprocess.run([sys.executable, "-c", "from pathlib import Path\n" + SCRIPT], capture_output=True, text=True, env=env,
                          timeout=900, cwd=str(root))
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    assert "debug build ok libms_kernels_dbg.so" in proc.stdout
