"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

A step runs only the tokens it is given, as one batch, from the cache that earlier steps left:
portions of prompts beside single decoded tokens, cut anywhere. It stands where the reference has
``ModelRunner.forward`` and ``forward_tokens`` (miniserve/engine/model_runner.py:220-315), with
one difference in what comes back: logits only at the places the caller asks for, instead of at
the last token of every row (miniserve/model/qwen3.py:183-186).
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, RequestCache
from ..ops import native
from ..parts.decoder import DecoderModel
from .context import StepContext


@dataclass
class StepRow:
    """One request's share of a step: its cache, its next tokens, and which of them (indices
    into ``tokens``) the caller wants logits for."""

    cache: RequestCache
    tokens: Sequence[int]
    want: Sequence[int] = ()
    # If set, the row brings one token that the host does not know yet: it is entry ``fill_from``
    # of the previous step's sampled tokens, still on the device (``tokens`` then holds any valid id).
    fill_from: int | None = None


def _leading_ones(q_len: np.ndarray, pad_rows: int, pad_len: int = 1) -> int:
    """How many rows from the front bring exactly one token (padding rows follow the real ones)."""
    other = np.flatnonzero(q_len != 1)
    return int(other[0]) if other.size else len(q_len) + (pad_rows if pad_len == 1 else 0)


class StepError(RuntimeError):
    pass


_NUM_BUFFERS = 3


class StepFunction:
    def __init__(self, model: DecoderModel, cache: CacheManager, arena_ints: int = 1 << 16):
        if model.device.type != "cuda":
            raise RuntimeError(
                "miniserve_b200 runs on a CUDA device only (there is no CPU implementation of the step function)")
        native.kernels()  # build / load now; raises if the kernels cannot be had
        self.model = model
        self.cache = cache
        self.device = model.device
        self.vocab_size = model.spec.vocab_size
        self._host_lib = native.host()
        self._arena_ints = 0
        self._pinned: list[torch.Tensor] = []
        self._events: list[torch.cuda.Event | None] = []
        self._dev_arena: torch.Tensor | None = None
        self._turn = 0
        self.arena_generation = 0  # bumped when the device arena moves (captured graphs become stale)
        self._grow(arena_ints)
        from .. import ops

        self.status = ops.device_status(self.device)  # shared by every kernel launched on this device
        props = torch.cuda.get_device_properties(self.device)
        self.sm_count = props.multi_processor_count
        self.persistent_scratch: dict = {}
        self.h2d_bytes = 0  # bytes of step metadata copied to the device so far
        # StepGraphs (engine/graphs.py) when the engine replays recurring step shapes from CUDA graphs; its
        # run() returns None for a step it does not take, which then runs eagerly
        self.graphs = None

    # ------------------------------------------------------------------ arena
    def _grow(self, ints: int) -> None:
        ints = max(ints, 1024)
        self._arena_ints = ints
        self._pinned = [torch.empty(ints, dtype=torch.int32, pin_memory=True) for _ in range(_NUM_BUFFERS)]
        self._events = [None] * _NUM_BUFFERS
        self._dev_arena = torch.empty(ints, dtype=torch.int32, device=self.device)
        self.arena_generation += 1

    def reserve_arena(self, ints: int) -> None:
        """Make the arena at least this large now, so that it does not move later."""
        if ints > self._arena_ints:
            torch.cuda.current_stream(self.device).synchronize()
            self._grow(ints)

    def _arena_need(self, rows: Sequence[StepRow], pad_rows: int, indices_cap: int = 0, pad_len: int = 1) -> int:
        t = sum(len(r.tokens) for r in rows) + pad_rows * pad_len
        r = len(rows) + pad_rows
        w = sum(len(x.want) for x in rows)
        pages = sum(sum(tb.num_entries + tb.blocks_needed(len(x.tokens)) for tb in x.cache.tables) for x in rows)
        groups = self.cache.num_groups
        pad_pages = pad_rows * -(-pad_len // self.cache.page_size)
        return (3 * (t + 4) + 4 * (r + 5) + (w + pad_rows + 4) + groups * (r + 5 + pad_pages + 4 + indices_cap)
                + pages + 64)

    # ------------------------------------------------------------------ the step
    def run(self, rows: Sequence[StepRow], pad_rows: int = 0, prev_tokens: torch.Tensor | None = None) -> torch.Tensor:
        """Run one step. Returns float32 logits ``[wanted, vocab]`` on the device, in the order
        of the rows and of each row's ``want``. Raises ``OutOfBlocks`` (nothing changed) if
        the pool cannot hold the step's new tokens."""
        logits = self.graphs.run(rows, prev_tokens) if self.graphs is not None and pad_rows == 0 else None
        if logits is None:
            ctx = self.prepare(rows, pad_rows, prev_tokens=prev_tokens)
            logits = self.model.forward(ctx, self.cache.entry_views)
        for r in rows:
            self.cache.trim(r.cache)
        return logits

    def prepare(self, rows: Sequence[StepRow], pad_rows: int = 0, indices_cap: int = 0,
                want_pad_rows: bool = False, prev_tokens: torch.Tensor | None = None, pad_len: int = 1) -> StepContext:
        """Reserve pages, pack the step and start its copy to the device. ``pad_rows`` adds
        padding rows (``pad_len`` tokens from position 0 on, on a page outside the allocator);
        ``indices_cap`` / ``want_pad_rows`` ask for the layout that depends on the padded row
        count alone (see ``csrc/host_core.cpp``), which captured graphs need."""
        if not rows:
            raise ValueError("a step needs at least one row")
        q_len = np.fromiter((len(r.tokens) for r in rows), dtype=np.int32, count=len(rows))
        if (q_len < 1).any():
            raise ValueError("every row of a step brings at least one token")
        q_start = np.fromiter((r.cache.num_tokens for r in rows), dtype=np.int32, count=len(rows))
        ids = np.concatenate([np.asarray(r.tokens, dtype=np.int64) for r in rows])
        if ids.min() < 0 or ids.max() >= self.vocab_size:
            raise ValueError(f"token id outside [0, {self.vocab_size})")
        ids = ids.astype(np.int32)
        want: list[int] = []
        base = 0
        for r, n in zip(rows, q_len):
            for w in r.want:
                if not 0 <= w < n:
                    raise IndexError(f"wanted place {w} outside the row's {n} tokens")
                want.append(base + int(w))
            base += int(n)
        want_arr = np.asarray(want, dtype=np.int32)
        slots = np.fromiter((r.cache.state_slot for r in rows), dtype=np.int32, count=len(rows))

        fills = [(i, r.fill_from) for i, r in enumerate(rows) if r.fill_from is not None]
        if fills:
            if prev_tokens is None or any(len(rows[i].tokens) != 1 for i, _ in fills):
                raise ValueError("a row filled from the previous step brings exactly one token and needs that step's tokens")
        need = self._arena_need(rows, pad_rows, indices_cap, pad_len) + 2 * len(fills) + 8
        if need > self._arena_ints:
            torch.cuda.current_stream(self.device).synchronize()
            self._grow(2 * need)
        # all-or-nothing page reservation, before anything else is touched
        self.cache.reserve([(r.cache, int(n)) for r, n in zip(rows, q_len)])

        groups = self.cache.num_groups
        tables = (ctypes.c_void_p * max(groups * len(rows), 1))()
        for g in range(groups):
            for i, r in enumerate(rows):
                tables[g * len(rows) + i] = r.cache.tables[g].handle
        pad_page = np.asarray([grp.pad_page for grp in self.cache.groups] or [0], dtype=np.int32)
        offsets = (ctypes.c_longlong * (9 + 2 * groups))()

        turn = self._turn
        self._turn = (turn + 1) % _NUM_BUFFERS
        if self._events[turn] is not None:
            self._events[turn].synchronize()  # the copy that last used this staging buffer is done
        pinned = self._pinned[turn]
        total = self._host_lib.ms_pack_step(
            pinned.data_ptr(), self._arena_ints, offsets, len(rows), pad_rows, q_start.ctypes.data,
            q_len.ctypes.data, ids.ctypes.data, slots.ctypes.data, want_arr.ctypes.data, len(want), groups, tables,
            pad_page.ctypes.data, indices_cap, int(want_pad_rows), self.cache.pad_state_slot, pad_len, self.cache.page_size)
        if total < 0:
            # undo the reservation so that a failed step leaves the tables as they were
            for r, n in zip(rows, q_len):
                for tb in r.cache.tables:
                    tb.rewind(int(n))
            native.host_check(int(-total))
        stream = torch.cuda.current_stream(self.device)
        dev = self._dev_arena
        packed = int(total)
        if fills:
            # (flat token index, entry of the previous step's tokens) pairs ride behind the packed step
            starts = np.concatenate(([0], np.cumsum(q_len)[:-1]))
            tail = np.asarray([starts[i] for i, _ in fills] + [src for _, src in fills], dtype=np.int32)
            pinned[packed:packed + tail.size] = torch.from_numpy(tail)
            total = packed + tail.size
        dev[:total].copy_(pinned[:total], non_blocking=True)
        self.h2d_bytes += int(total) * 4
        if fills:
            k = native.kernels()
            native.kernel_check(k.ms_fill_tokens(dev[int(offsets[0]):].data_ptr(), dev[packed:].data_ptr(), prev_tokens.data_ptr(),
                                                 dev[packed + len(fills):].data_ptr(), len(fills), stream.cuda_stream))
            total = packed
        ev = torch.cuda.Event()
        ev.record(stream)
        self._events[turn] = ev

        t_all = int(q_len.sum()) + pad_rows * pad_len
        r_all = len(rows) + pad_rows
        o = list(offsets)

        def view(start: int, n: int) -> torch.Tensor:
            return dev[start:start + n]

        page_indptr, page_indices = [], []
        for g in range(groups):
            page_indptr.append(view(o[8 + 2 * g], r_all + 1))
            end = o[8 + 2 * g + 2] if g + 1 < groups else total
            page_indices.append(view(o[9 + 2 * g], max(end - o[9 + 2 * g], 1)))
        kv_end = q_start + q_len
        return StepContext(
            num_tokens=t_all, num_rows=r_all, num_logit_rows=len(want) + (pad_rows if want_pad_rows else 0),
            stream=stream.cuda_stream,
            token_ids=view(o[0], t_all), positions=view(o[1], t_all), row_of_token=view(o[2], t_all),
            cu_q=view(o[3], r_all + 1), q_start=view(o[4], r_all), kv_len=view(o[5], r_all),
            state_slot=view(o[6], r_all),
            logit_rows=view(o[7], max(len(want) + (pad_rows if want_pad_rows else 0), 1)),
            page_indptr=page_indptr, page_indices=page_indices, status=self.status,
            host_q_start=q_start.tolist() + [0] * pad_rows, host_q_len=q_len.tolist() + [pad_len] * pad_rows,
            host_state_slot=slots.tolist() + [self.cache.pad_state_slot] * pad_rows,
            max_q_len=max(int(q_len.max()), pad_len if pad_rows else 1), max_kv_len=max(int(kv_end.max()), pad_len if pad_rows else 1),
            decode_only=bool((q_len == 1).all()),
            leading_single_rows=_leading_ones(q_len, pad_rows, pad_len), sm_count=self.sm_count, scratch=self.persistent_scratch,
            layout=tuple(o))

    def reset_after_fault(self) -> None:
        """After a kernel raised the status word: wait for what is in flight, then zero the word and
        the kernels' persistent counters. A kernel that gave up may have left its tickets, work-queue
        counters or barrier state half counted; they go back to zero in place, because CUDA graphs
        hold their addresses."""
        torch.cuda.current_stream(self.device).synchronize()
        self.status.zero_()
        for buf in self.persistent_scratch.values():
            if isinstance(buf, torch.Tensor) and buf.dtype == torch.int32:
                buf.zero_()

    def check_status(self) -> None:
        """Synchronise and raise if a kernel flagged inconsistent input (a page that was given
        back, a table too short)."""
        code = int(self.status.item())
        if code:
            self.reset_after_fault()
            raise StepError(f"a kernel reported a fault it caught itself (code {code}: 2-3 inconsistent cache "
                            f"metadata; 11-13, 21-24, 31-34 a bounded wait in a tensor-core pipeline ran out)")
