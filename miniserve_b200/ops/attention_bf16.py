"""bfloat16 tensor-core attention (``csrc/attention_bf16.cu``), compiled per head size on first
use: a model only pays for the head size it has."""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_void_p
from functools import lru_cache

import torch

from . import build, native

_p, _i, _f = c_void_p, c_int, c_float


def _flag(name: str, default: str) -> bool:
    import os

    return os.environ.get(name, default) == "1"


CLUSTER_MERGE = _flag("MINISERVE_CLUSTER_MERGE", "1")  # 2 to 8 key splits of a decode step as one thread-block cluster


def supports(head_dim: int, page_size: int) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= 256 and page_size & (page_size - 1) == 0


def module_for(head_dim: int) -> build.Module:
    return build.Module(f"attn_bf16_d{head_dim}", ("attention_bf16.cu",), defines=(f"MS_HEAD_DIM={head_dim}",))


@lru_cache(maxsize=None)
def _lib(head_dim: int):
    if not supports(head_dim, 16):
        raise ValueError(f"the bfloat16 attention kernels take head sizes that are multiples of 16 up to 256, not {head_dim}")
    lib = ctypes.CDLL(str(build.ensure_built(module_for(head_dim))))
    pre = f"ms_attn_bf16_d{head_dim}_"
    fns = {}
    for name, args, res in (
        ("last_error", [], c_char_p),
        ("prefill", [_p] * 8 + [_i, _i, _i, _i, _f, _i, _i, _p], c_int),
        ("decode", [_p] * 9 + [_i, _i, _i, _f, _i, _i, _i, _p], c_int),
        ("decode_fused", [_p] * 10 + [_i, _i, _i, _f, _i, _i, _i, _p], c_int),
        ("decode_cluster", [_p] * 7 + [_i, _i, _i, _f, _i, _i, _i, _p], c_int),
        ("decode_clusters_resident", [_i, ctypes.POINTER(c_int)], c_int),
    ):
        fn = getattr(lib, pre + name)
        fn.argtypes, fn.restype = args, res
        fns[name] = fn
    set_pdl = getattr(lib, pre + "set_pdl")
    set_pdl.argtypes, set_pdl.restype = [c_int], None
    set_pdl(int(native.pdl_enabled()))
    fns["lib"] = lib
    return fns


def _check(fns, rc: int, launches: int = 1) -> None:
    native.LAUNCHES[0] += launches
    if rc != 0:
        raise native.NativeError(fns["last_error"]().decode())


@lru_cache(maxsize=None)
def clusters_resident(head_dim: int, splits: int, device_index: int = 0) -> int:
    """How many thread-block clusters of ``splits`` decode CTAs the device holds at a time (a cluster
    lies within one GPC: on a B200 with head size 128, 71 clusters of 4 and 33 of 8, not 74 and 37)."""
    fns = _lib(head_dim)
    out = c_int(0)
    with torch.cuda.device(device_index):
        rc = fns["decode_clusters_resident"](splits, ctypes.byref(out))
    if rc != 0:
        raise native.NativeError(fns["last_error"]().decode())
    return out.value


def choose_splits(rows: int, head_chunks: int, max_kv_len: int | None, sm_count: int, resident=None) -> int:
    """How many ways the keys of each (request, kv head) are split across CTAs: as many as give
    one wave of two CTAs per SM, but at least 128 keys per split and at most 16 splits up to 4,096 keys
    (measured on B200 at contexts of 512 to 4,096 and batches of 1 to 32: more splits only add partial
    results to merge, fewer leave SMs idle; one split too many and the CTAs no longer fit one wave: a
    decode step of 8 requests at 2,048 tokens takes 1.28 ms with 4 splits, 1.34 with 3, 1.60 with 8).
    Beyond that a split is not asked to walk more than 256 keys while CTAs would be idle: a single
    request of 8,192 keys is cut 32 ways, of 32,768 keys 37 ways (every CTA that fits): 1.33 -> 1.15 ms
    per step at 8,192 keys, 2.83 -> 1.60 at 32,768, 9.01 -> 3.43 at 131,072 (4.7 TB/s).
    ``max_kv_len`` None (inside a CUDA graph for short contexts, where the launch cannot follow the
    context length): assume a few thousand keys, and stay within the 8 splits that one thread-block
    cluster merges (a single request: 0.98 ms per step with 8 splits, 0.99 with 16).
    ``resident(splits)``: how many clusters of that size the device holds at a time; splits that run
    as a cluster (2 to 8) are reduced until every (request, head group) has its cluster in the first
    wave (6 requests x 8 head groups in clusters of 6: 48 clusters where 45 fit, and the step took 1.33 ms
    against 1.17 for 8 requests in clusters of 4). A few more than 8 splits are not worth leaving the
    cluster for: 9 to 11 become 8."""
    items = max(rows * head_chunks, 1)
    want = (2 * sm_count) // items
    by_len = 8 if max_kv_len is None else max(1, -(-max_kv_len // 128))
    most = 16 if max_kv_len is None else max(16, max_kv_len // 256)
    splits = max(1, min(want, by_len, most))
    if 8 < splits < 12:
        splits = 8
    if resident is not None:
        while 2 <= splits <= 8 and resident(splits) < items:
            splits -= 1
    return splits


def _scratch(ctx, rows: int, nq: int, splits: int, d: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    need = rows * nq * splits
    if ctx.graph_bucket:
        # inside a CUDA graph capture: memory of the graph's own pool, alive as long as the graph
        return (torch.empty(need * d, dtype=torch.float32, device=device),
                torch.empty(need * 2, dtype=torch.float32, device=device))
    buf = ctx.scratch.get("attn_decode")
    if buf is None or buf[0].numel() < need * d or buf[1].numel() < need * 2:
        buf = (torch.empty(need * d, dtype=torch.float32, device=device),
               torch.empty(need * 2, dtype=torch.float32, device=device))
        ctx.scratch["attn_decode"] = buf
    return buf


def run(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, ctx, group: int,
        scale: float, window: int | None) -> None:
    """The step's attention: rows at the front that bring one token each go to the split-key
    decode kernel, the rest to the tiled kernel."""
    single = ctx.leading_single_rows
    if single:
        run_decode(out, q, k_pool, v_pool, ctx, group, scale, window, single)
    if single < ctx.num_rows:
        run_prefill(out, q, k_pool, v_pool, ctx, group, scale, window, single)


def run_decode(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, ctx, group: int,
               scale: float, window: int | None, rows: int) -> None:
    """Rows [0, rows) of the step, one new token each (so token i belongs to row i): keys split
    across CTAs, partial results merged by the last CTA of each (row, head group) to finish."""
    t, nq, d = q.shape
    nkv, page_size = k_pool.shape[1], k_pool.shape[2]
    fns = _lib(d)
    indptr, indices = ctx.page_indptr[group], ctx.page_indices[group]
    chunks = nkv * -(-(nq // nkv) // 16)
    fit = (lambda n: clusters_resident(d, n, q.device.index or 0)) if CLUSTER_MERGE else None
    known = ctx.max_kv_len if not ctx.graph_bucket else (getattr(ctx, "graph_kv_len", 0) or None)
    splits = choose_splits(rows, chunks, known, ctx.sm_count, fit)
    if CLUSTER_MERGE and 2 <= splits <= 8:
        # the splits as one thread-block cluster: merged through distributed shared memory
        _check(fns, fns["decode_cluster"](
            out.data_ptr(), q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), ctx.kv_len.data_ptr(), indptr.data_ptr(),
            indices.data_ptr(), rows, nq, nkv, float(scale), int(window or 0), page_size, splits, ctx.stream))
        return
    part_o = part_ml = counters = None
    if splits > 1:
        part_o, part_ml = _scratch(ctx, rows, nq, splits, d, q.device)
        counters = ctx.scratch.get("attn_counters")
        if counters is None or counters.numel() < rows * chunks:
            # tickets of the fused merge: zero before the first launch, left zero by every launch
            if counters is not None:  # captured graphs may hold the smaller one's address: it stays alive
                ctx.scratch.setdefault("retired", []).append(counters)
            counters = torch.zeros(max(4096, rows * chunks), dtype=torch.int32, device=q.device)
            ctx.scratch["attn_counters"] = counters
    _check(fns, fns["decode_fused"](
        out.data_ptr(), None if part_o is None else part_o.data_ptr(), None if part_ml is None else part_ml.data_ptr(),
        None if counters is None else counters.data_ptr(), q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), ctx.kv_len.data_ptr(), indptr.data_ptr(),
        indices.data_ptr(), rows, nq, nkv, float(scale), int(window or 0), page_size, splits, ctx.stream),
        launches=1)


def run_prefill(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, ctx, group: int,
                scale: float, window: int | None, first_row: int = 0) -> None:
    """Rows [first_row, num_rows) of the step, any number of new tokens each: tiles of 64 queries
    over the row's pages (``mma.sync``; the tcgen05 kernel of ``attention_tc.cu`` takes head size 128)."""
    t, nq, d = q.shape
    nkv, page_size = k_pool.shape[1], k_pool.shape[2]
    fns = _lib(d)
    indptr, indices = ctx.page_indptr[group], ctx.page_indices[group]
    skip = 4 * first_row  # the per-row tables are int32
    _check(fns, fns["prefill"](
        out.data_ptr(), q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), ctx.cu_q.data_ptr() + skip, ctx.q_start.data_ptr() + skip,
        indptr.data_ptr() + skip, indices.data_ptr(), ctx.num_rows - first_row, ctx.max_q_len, nq, nkv, float(scale), int(window or 0),
        page_size, ctx.stream))
