"""Python faces of the C++ block allocator and block table (``csrc/host_core.cpp``).

Same contract as miniserve/cache/block_allocator.py and block_table.py: allocation order is
part of the contract (fresh: 0, 1, 2, ...; freed blocks are reused last-in first-out),
``allocate`` is all-or-nothing, ``free`` validates the whole call before it changes anything.
"""

from __future__ import annotations

import ctypes
from typing import Iterable, Sequence

from ..ops import native
from ..ops.native import OutOfBlocks, host_check

__all__ = ["BlockAllocator", "BlockTable", "OutOfBlocks"]


def _ints(values: Iterable[int]):
    values = list(values)
    return (ctypes.c_int32 * len(values))(*values), len(values)


class BlockAllocator:
    def __init__(self, num_blocks: int, block_size: int):
        self._lib = native.host()
        self._h = self._lib.ms_alloc_create(int(num_blocks), int(block_size))
        if not self._h:
            raise ValueError(self._lib.ms_host_last_error().decode())
        self.num_blocks = int(num_blocks)
        self.block_size = int(block_size)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.ms_alloc_destroy(h)

    @property
    def num_free(self) -> int:
        return self._lib.ms_alloc_num_free(self._h)

    @property
    def num_used(self) -> int:
        return self.num_blocks - self.num_free

    def can_allocate(self, n: int) -> bool:
        return 0 <= n <= self.num_free

    def refcount(self, block: int) -> int:
        out = ctypes.c_int()
        host_check(self._lib.ms_alloc_refcount(self._h, int(block), ctypes.byref(out)))
        return out.value

    def allocate(self, n: int) -> list[int]:
        buf = (ctypes.c_int32 * max(int(n), 1))()
        host_check(self._lib.ms_alloc_allocate(self._h, int(n), buf))
        return list(buf[:n])

    def incref(self, blocks: Iterable[int]) -> None:
        arr, n = _ints(blocks)
        host_check(self._lib.ms_alloc_incref(self._h, arr, n))

    def free(self, blocks: Iterable[int]) -> None:
        arr, n = _ints(blocks)
        host_check(self._lib.ms_alloc_free(self._h, arr, n))

    def new_table(self) -> "BlockTable":
        return BlockTable(self)

    def check_invariants(self) -> None:
        if self._lib.ms_alloc_check(self._h) != 0:
            raise AssertionError(self._lib.ms_host_last_error().decode())


class BlockTable:
    """Token position -> page of one request in one cache group."""

    def __init__(self, allocator: BlockAllocator):
        self.allocator = allocator
        self.block_size = allocator.block_size
        self._lib = allocator._lib
        self._h = self._lib.ms_table_create(allocator._h)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.ms_table_destroy(h)

    @property
    def handle(self) -> int:
        return self._h

    @property
    def num_tokens(self) -> int:
        return self._lib.ms_table_num_tokens(self._h)

    @property
    def num_entries(self) -> int:
        """Pages the table has ever covered, including those given back (which read -1)."""
        return self._lib.ms_table_num_entries(self._h)

    @property
    def num_blocks(self) -> int:
        """Pages the table holds now."""
        return self._lib.ms_table_num_held(self._h)

    @property
    def blocks(self) -> list[int]:
        n = self.num_entries
        buf = (ctypes.c_int32 * max(n, 1))()
        host_check(self._lib.ms_table_copy_blocks(self._h, buf, n))
        return list(buf[:n])

    @property
    def capacity(self) -> int:
        return self.num_entries * self.block_size

    def blocks_needed(self, n: int) -> int:
        out = ctypes.c_int()
        host_check(self._lib.ms_table_blocks_needed(self._h, int(n), ctypes.byref(out)))
        return out.value

    def append_tokens(self, n: int) -> None:
        host_check(self._lib.ms_table_append_tokens(self._h, int(n)))

    def slot(self, pos: int) -> int:
        out = ctypes.c_longlong()
        host_check(self._lib.ms_table_slot(self._h, int(pos), ctypes.byref(out)))
        return out.value

    def rewind(self, n: int) -> None:
        host_check(self._lib.ms_table_rewind(self._h, int(n)))

    def release(self) -> None:
        host_check(self._lib.ms_table_release(self._h))

    def release_below(self, pos: int) -> int:
        """Give back the pages that lie wholly below position ``pos``; returns how many."""
        out = ctypes.c_int()
        host_check(self._lib.ms_table_release_below(self._h, int(pos), ctypes.byref(out)))
        return out.value
