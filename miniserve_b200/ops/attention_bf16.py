"""bfloat16 tensor-core attention kernels (compiled per head size on first use)."""

from __future__ import annotations


def supports(head_dim: int, page_size: int) -> bool:
    return False


def run(out, q, k_pool, v_pool, ctx, group, scale, window) -> None:
    raise NotImplementedError
