"""The cache manager: pages of keys and values in groups, block tables per request, and
slots for per-request state of fixed size.

The reference keeps one pool tensor for all layers and one table per request
(miniserve/cache/kv_pool.py:14-50, miniserve/cache/kv_cache.py:33-136 with the prefix cache
switched off). Here run entries with the same need (kv heads, head size, window) form a
*group*; each group has pages, an allocator and per-request tables of its own, because a group
that only looks a window back gives pages back while a request is still running, and a group
that keeps every key does not. Pages return to their allocator when a request ends or is
preempted (``release``), when an admission is refused, and, for a windowed group, as soon as
the window has passed them (``trim``). A failed ``reserve`` changes nothing.

Beside the pages there are slots for per-request state of fixed size: one slot id per live
request, indexing a tensor per run entry that declared such state. Qwen3 declares none, so
the tensors are absent and only the slot ids are handed out.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import torch

from ..parts.base import FixedState, PagedKV
from ..parts.decoder import EntryCache
from .blocks import BlockAllocator, BlockTable, OutOfBlocks


@dataclass
class CacheGroup:
    need: PagedKV
    entries: list[int]  # run entries that own a cache in this group
    allocator: BlockAllocator
    page_size: int
    k: torch.Tensor | None = None  # [entries, pages + 1, kv_heads, page_size, head_dim]
    v: torch.Tensor | None = None

    @property
    def pad_page(self) -> int:
        """A page outside the allocator, written and read only by padding rows."""
        return self.allocator.num_blocks

    def bytes_per_token(self, itemsize: int) -> int:
        return 2 * len(self.entries) * self.need.kv_heads * self.need.head_dim * itemsize


@dataclass
class KVEntryView:
    """What an attention mixer gets: its group's index (to pick the page table from the step
    context), its own K and V pools [pages + 1, kv_heads, page_size, head_dim]."""

    group: int
    k: torch.Tensor | None
    v: torch.Tensor | None
    page_size: int


@dataclass
class StateEntryView:
    """What a mixer with fixed-size state gets: ``state[slot]`` belongs to the request whose
    slot id is ``ctx.state_slot[row]``. The tensor has one slot more than the cache has requests:
    the padding rows of a captured graph carry that slot's id, so a mixer needs no mask for them."""

    state: torch.Tensor | None
    shape: tuple[int, ...]


@dataclass
class RequestCache:
    """Everything one live request holds: a table per group and a state slot."""

    tables: list[BlockTable]
    state_slot: int = -1
    released: bool = False

    @property
    def num_tokens(self) -> int:
        return self.tables[0].num_tokens if self.tables else self._tokens_without_tables

    _tokens_without_tables: int = 0


def group_needs(entry_caches: Sequence[EntryCache]) -> tuple[list[tuple[PagedKV, int]], list[FixedState]]:
    """What a model's run entries ask of the cache: ``[(need, number of entries)]`` for the paged
    groups (entries with equal needs share a group), and the fixed-size states, one per owning
    entry. The order of the groups is the one ``CacheManager`` uses."""
    groups: dict[PagedKV, int] = {}
    states: list[FixedState] = []
    for i, ec in enumerate(entry_caches):
        if ec.owner != i or ec.need is None:
            continue
        if isinstance(ec.need, PagedKV):
            groups[ec.need] = groups.get(ec.need, 0) + 1
        elif isinstance(ec.need, FixedState):
            states.append(ec.need)
    return list(groups.items()), states


def window_pages(window: int, page_size: int, step_tokens: int) -> int:
    """The most pages a request holds in a group that looks ``window`` keys back, when a step brings
    it at most ``step_tokens`` tokens: the window and the step's tokens (pages are given back after
    the step), plus the pages both ends cut into."""
    return -(-(window + step_tokens) // page_size) + 1


class CacheManager:
    def __init__(self, entry_caches: Sequence[EntryCache], num_pages: "int | Sequence[int]", page_size: int, max_requests: int,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device | str | None = None,
                 poison: bool = False, poison_on_free: bool = False, step_tokens: int | None = None):
        """``entry_caches``: one per run entry (``DecoderModel.entry_caches``). ``num_pages``:
        pages of ``page_size`` tokens, one number for every group or one per group (in the order
        of ``group_needs``). ``device`` None keeps everything on the host (bookkeeping only, for
        tests). ``poison`` fills the pools with NaN so that a read of a slot nobody wrote shows
        up; ``poison_on_free`` also fills a request's pages with NaN when it gives them back, so
        that a stale key read through a reused page shows up (a debugging aid: it launches a fill
        per release). ``step_tokens``: the most tokens a step brings one request; with it,
        ``pages_for`` knows that a windowed group never holds a whole long request."""
        if page_size < 1 or page_size & (page_size - 1):
            raise ValueError(f"page_size must be a power of two, got {page_size}")
        needs, _ = group_needs(entry_caches)
        per_group = [int(num_pages)] * len(needs) if isinstance(num_pages, int) else [int(n) for n in num_pages]
        if len(per_group) != len(needs):
            raise ValueError(f"{len(per_group)} page counts for {len(needs)} cache groups")
        if any(n < 1 for n in per_group) or (isinstance(num_pages, int) and num_pages < 1):
            raise ValueError(f"the pool needs at least one page, got {num_pages}")
        self.page_size = page_size
        self.num_pages = max(per_group) if per_group else (num_pages if isinstance(num_pages, int) else 0)
        self.step_tokens = step_tokens
        self.poison_on_free = poison_on_free
        self.max_requests = max_requests
        self.dtype = dtype
        self.device = torch.device(device) if device is not None else None
        self.groups: list[CacheGroup] = []
        self._entry_view: list[KVEntryView | StateEntryView | None] = []
        self._state_entries: list[tuple[int, FixedState]] = []
        by_need: dict[PagedKV, int] = {}
        owners: dict[int, tuple[int, int]] = {}  # owner entry -> (group, index in group)
        for i, ec in enumerate(entry_caches):
            if ec.owner != i or ec.need is None:
                continue
            if isinstance(ec.need, PagedKV):
                g = by_need.get(ec.need)
                if g is None:
                    g = len(self.groups)
                    by_need[ec.need] = g
                    self.groups.append(CacheGroup(ec.need, [], BlockAllocator(per_group[g], page_size), page_size))
                owners[i] = (g, len(self.groups[g].entries))
                self.groups[g].entries.append(i)
            elif isinstance(ec.need, FixedState):
                self._state_entries.append((i, ec.need))
            else:
                raise TypeError(f"run entry {i} asks for an unknown kind of cache: {ec.need!r}")
        if self.device is not None:
            for grp in self.groups:
                shape = (len(grp.entries), grp.allocator.num_blocks + 1, grp.need.kv_heads, page_size, grp.need.head_dim)
                fill = float("nan") if poison else 0.0
                grp.k = torch.full(shape, fill, dtype=dtype, device=self.device)
                grp.v = torch.full(shape, fill, dtype=dtype, device=self.device)
        state_tensors: dict[int, torch.Tensor | None] = {}
        for i, need in self._state_entries:
            # one slot more than there are requests: the padding rows of a captured graph read and write it
            state_tensors[i] = (torch.zeros((max_requests + 1, *need.shape), dtype=need.dtype, device=self.device)
                                if self.device is not None else None)
        for i, ec in enumerate(entry_caches):
            if ec.need is None:
                self._entry_view.append(None)
            elif isinstance(ec.need, PagedKV):
                g, idx = owners[ec.owner]
                grp = self.groups[g]
                self._entry_view.append(KVEntryView(g, grp.k[idx] if grp.k is not None else None,
                                                    grp.v[idx] if grp.v is not None else None, page_size))
            else:
                self._entry_view.append(StateEntryView(state_tensors[ec.owner], tuple(ec.need.shape)))
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self._live: set[int] = set()

    # ------------------------------------------------------------------ views and sizes
    @property
    def pad_state_slot(self) -> int:
        """A state slot outside the ones requests get, for padding rows (as ``pad_page`` is for pages)."""
        return self.max_requests

    @property
    def entry_views(self) -> list:
        return self._entry_view

    @property
    def num_groups(self) -> int:
        return len(self.groups)

    def bytes_per_token(self) -> int:
        item = torch.empty((), dtype=self.dtype).element_size()
        return sum(g.bytes_per_token(item) for g in self.groups)

    def pool_bytes(self) -> int:
        return sum(g.k.numel() * g.k.element_size() * 2 for g in self.groups if g.k is not None)

    def state_bytes(self) -> int:
        """Bytes of the per-request state tensors (one slot per request the cache can hold)."""
        return sum(v.state.numel() * v.state.element_size() for v in self._entry_view
                   if isinstance(v, StateEntryView) and v.state is not None)

    # ------------------------------------------------------------------ requests
    def new_request(self) -> RequestCache:
        """Empty tables and a state slot for a request that is being admitted."""
        if not self._free_slots:
            raise OutOfBlocks(f"all {self.max_requests} request slots are taken")
        slot = self._free_slots.pop()
        self._live.add(slot)
        return RequestCache([g.allocator.new_table() for g in self.groups], slot)

    def release(self, rc: RequestCache) -> None:
        """Give back everything ``rc`` holds (request finished, aborted, preempted or refused)."""
        if rc.released:
            raise ValueError("request cache released twice")
        if self.poison_on_free and self.device is not None:
            for g, t in zip(self.groups, rc.tables):
                held = [b for b in t.blocks if b >= 0]
                if held and g.k is not None:
                    idx = torch.tensor(held, dtype=torch.long, device=self.device)
                    g.k[:, idx] = float("nan")
                    g.v[:, idx] = float("nan")
        for t in rc.tables:
            t.release()
        if rc.state_slot >= 0:
            self._live.discard(rc.state_slot)
            self._free_slots.append(rc.state_slot)
        rc.state_slot = -1
        rc.released = True

    @property
    def num_free_slots(self) -> int:
        return len(self._free_slots)

    # ------------------------------------------------------------------ page budget
    def num_free(self) -> tuple[int, ...]:
        return tuple(g.allocator.num_free for g in self.groups)

    def pages_for(self, num_tokens: int) -> tuple[int, ...]:
        """Pages per group that a request of ``num_tokens`` tokens may hold at its largest: all of
        them, or, in a windowed group (when the step size is known), the window and a step's tokens."""
        out = []
        for g in self.groups:
            n = -(-num_tokens // g.page_size)
            if g.need.window and self.step_tokens:
                n = min(n, window_pages(g.need.window, g.page_size, self.step_tokens))
            out.append(n)
        return tuple(out)

    def group_pages(self) -> tuple[int, ...]:
        """Pages each group's pool has."""
        return tuple(g.allocator.num_blocks for g in self.groups)

    def pages_needed(self, rc: RequestCache, new_tokens: int) -> tuple[int, ...]:
        """Pages per group that appending ``new_tokens`` to ``rc`` would allocate."""
        return tuple(t.blocks_needed(new_tokens) for t in rc.tables)

    def pages_held(self, rc: RequestCache) -> tuple[int, ...]:
        """Pages per group that ``rc`` holds now (a windowed group has given the older ones back)."""
        return tuple(t.num_blocks for t in rc.tables)

    def pages_outstanding(self, rc: RequestCache, upto_tokens: int) -> tuple[int, ...]:
        """Pages per group that ``rc`` may still take, net of what it gives back, before its
        sequence reaches ``upto_tokens`` tokens: the pages not yet allocated, but in a windowed
        group (when the step size is known) no more than brings it to the most it ever holds."""
        out = []
        for g, t in zip(self.groups, rc.tables):
            n = max(0, -(-upto_tokens // g.page_size) - t.num_entries)
            if g.need.window and self.step_tokens:
                n = min(n, max(0, window_pages(g.need.window, g.page_size, self.step_tokens) - t.num_blocks))
            out.append(n)
        return tuple(out)

    def fits(self, need: Sequence[int], margin: Sequence[int] | None = None) -> bool:
        free = self.num_free()
        margin = margin or (0,) * len(free)
        return all(n <= f - m for n, f, m in zip(need, free, margin))

    def reserve(self, rows: Sequence[tuple[RequestCache, int]]) -> None:
        """Extend every row's tables by its new tokens. All or nothing: if any group is short,
        raise ``OutOfBlocks`` with every table as it was (miniserve/engine/model_runner.py:309-315)."""
        for gi, g in enumerate(self.groups):
            need = sum(rc.tables[gi].blocks_needed(n) for rc, n in rows)
            if need > g.allocator.num_free:
                raise OutOfBlocks(f"need {need} free pages in cache group {gi}, {g.allocator.num_free} free")
        for rc, n in rows:
            if rc.released:
                raise ValueError("reserve on a released request cache")
            for t in rc.tables:
                t.append_tokens(n)
            rc._tokens_without_tables += n

    def trim(self, rc: RequestCache) -> int:
        """After a step: give back the pages of windowed groups that no later query can reach.
        The next query sits at position ``num_tokens`` and sees keys from
        ``num_tokens - window + 1`` on. Returns the number of pages freed."""
        freed = 0
        for g, t in zip(self.groups, rc.tables):
            if g.need.window:
                freed += t.release_below(t.num_tokens - g.need.window + 1)
        return freed

    # ------------------------------------------------------------------ checks
    def check_invariants(self) -> None:
        for g in self.groups:
            g.allocator.check_invariants()
        assert len(set(self._free_slots)) == len(self._free_slots), "a state slot is free twice"
        assert not (set(self._free_slots) & self._live), "a state slot is both free and live"
        assert len(self._free_slots) + len(self._live) == self.max_requests, "a state slot was lost"

    def is_idle(self) -> bool:
        """Nothing held by anyone: every page and every slot is free."""
        return all(g.allocator.num_free == g.allocator.num_blocks for g in self.groups) and not self._live
