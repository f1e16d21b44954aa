"""Helpers of the kernel tests: scatter contiguous keys/values into a paged pool and build the
flat step metadata by hand (independently of the product's packer)."""

from __future__ import annotations

import random

import torch


class PagedBatch:
    """Rows of (start, q_len) over random non-contiguous pages. Builds, on the device:
    positions, row_of_token, page_indptr, page_indices, and fills K/V pools
    [pages, kv_heads, page_size, d] from per-row contiguous k, v [kv_len, kv_heads, d]."""

    def __init__(self, rows: list[tuple[int, int]], page_size: int, kv_heads: int, d: int, dtype, seed: int = 0,
                 spare_pages: int = 5, device="cuda", share: "PagedBatch | None" = None):
        """``share``: reuse another batch's tables and pools (a later step of the same requests)."""
        rng = random.Random(seed)
        self.rows, self.page_size = rows, page_size
        need = [-(-(s + n) // page_size) for s, n in rows]
        if share is not None:
            self.tables = [t[:n] for t, n in zip(share.tables, need)]
            assert all(len(t) == n for t, n in zip(self.tables, need)), "the shared tables are too short"
            self.num_pages, self.k_pool, self.v_pool = share.num_pages, share.k_pool, share.v_pool
        else:
            total = sum(need) + spare_pages
            order = list(range(total))
            rng.shuffle(order)
            self.tables, at = [], 0
            for n in need:
                self.tables.append(order[at:at + n])
                at += n
            self.num_pages = total
            self.k_pool = torch.full((total, kv_heads, page_size, d), float("nan"), dtype=dtype, device=device)
            self.v_pool = torch.full_like(self.k_pool, float("nan"))
        pos, row_of = [], []
        for r, (s, n) in enumerate(rows):
            pos += list(range(s, s + n))
            row_of += [r] * n
        i32 = dict(dtype=torch.int32, device=device)
        self.positions = torch.tensor(pos, **i32)
        self.row_of_token = torch.tensor(row_of, **i32)
        indptr = [0]
        for t in self.tables:
            indptr.append(indptr[-1] + len(t))
        self.page_indptr = torch.tensor(indptr, **i32)
        self.page_indices = torch.tensor([p for t in self.tables for p in t], **i32)
        self.cu_q = torch.tensor([0] + list(torch.tensor([n for _, n in rows]).cumsum(0)), **i32)
        self.q_start = torch.tensor([s for s, _ in rows], **i32)
        self.kv_len = torch.tensor([s + n for s, n in rows], **i32)
        self.status = torch.zeros(1, **i32)
        self.num_tokens = len(pos)

    def fill(self, row: int, k: torch.Tensor, v: torch.Tensor, upto: int | None = None) -> None:
        """Write k, v [len, kv_heads, d] of ``row`` (positions 0..len-1, or ..upto-1) into its pages."""
        n = k.shape[0] if upto is None else upto
        for p in range(n):
            page = self.tables[row][p // self.page_size]
            self.k_pool[page, :, p % self.page_size] = k[p]
            self.v_pool[page, :, p % self.page_size] = v[p]

    def read(self, row: int, pool: torch.Tensor, n: int) -> torch.Tensor:
        out = []
        for p in range(n):
            page = self.tables[row][p // self.page_size]
            out.append(pool[page, :, p % self.page_size])
        return torch.stack(out)


def reference_attention(q, k, v, q_positions, scale, window=None):
    """Plain float32 attention of queries at absolute positions over keys 0..len-1 of one request.
    q: [n, heads, d]; k, v: [len, kv_heads, d]."""
    n, heads, d = q.shape
    group = heads // k.shape[1]
    out = torch.empty((n, heads, d), dtype=torch.float32, device=q.device)
    kpos = torch.arange(k.shape[0], device=q.device)
    for i in range(n):
        p = int(q_positions[i])
        ok = kpos <= p
        if window:
            ok &= kpos > p - window
        for h in range(heads):
            s = (k[:, h // group].float() @ q[i, h].float()) * scale
            s = s.masked_fill(~ok, float("-inf"))
            out[i, h] = torch.softmax(s, 0) @ v[:, h // group].float()
    return out


def make_context(pb: PagedBatch, logit_rows=None, device="cuda"):
    """A StepContext built by hand from a PagedBatch (independently of the product's packer)."""
    from miniserve_b200.engine.context import StepContext

    lr = torch.tensor(logit_rows if logit_rows is not None else [0], dtype=torch.int32, device=device)
    props = torch.cuda.get_device_properties(0)
    return StepContext(
        num_tokens=pb.num_tokens, num_rows=len(pb.rows), num_logit_rows=len(logit_rows or []),
        stream=torch.cuda.current_stream().cuda_stream, token_ids=None, positions=pb.positions,
        row_of_token=pb.row_of_token, cu_q=pb.cu_q, q_start=pb.q_start, kv_len=pb.kv_len,
        state_slot=torch.full((len(pb.rows),), -1, dtype=torch.int32, device=device), logit_rows=lr,
        page_indptr=[pb.page_indptr], page_indices=[pb.page_indices], status=pb.status,
        host_q_start=[s for s, _ in pb.rows], host_q_len=[n for _, n in pb.rows],
        host_state_slot=[-1] * len(pb.rows),
        max_q_len=max(n for _, n in pb.rows), max_kv_len=max(s + n for s, n in pb.rows),
        decode_only=all(n == 1 for _, n in pb.rows),
        leading_single_rows=next((i for i, (_, n) in enumerate(pb.rows) if n != 1), len(pb.rows)),
        sm_count=props.multi_processor_count)
