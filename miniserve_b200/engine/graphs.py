"""CUDA graphs: for decode-only steps (``DecodeGraphs``) and for other steps whose shape comes again
(``StepGraphs``, at the end of this file).

A decode step of a small model is launch-bound: a few hundred short kernels. The reference
captures one graph per batch-size bucket and pads a step up to its bucket with rows that write
a page outside the allocator (miniserve/engine/cuda_graph.py:49-274). The same is done here:
buckets are the powers of two up to the largest batch, and that batch itself, and between two powers
from 16 on the size halfway (24, 48, 96, ...: measured at Qwen3-0.6B sizes, 20 requests at 2,048 tokens
take 2.07 ms per step padded to 24 rows against 2.28 padded to 32, 40 requests 3.46 against 3.75; below
16 the halfway sizes gain nothing, the attention kernel's key splits being what they are for the next
power of two); a graph holds the
whole forward pass and the sampling kernel; the step's metadata is packed on the host and
copied into a fixed device arena before the replay, so nothing inside the graph moves.
Graphs are captured on first use of their bucket. A bucket has a graph for each class of context
length (the longest row's: below 8,192 keys, from 8,192, from 32,768, from 131,072), because the
attention kernel's launch inside a graph cannot follow the lengths: a graph for short contexts cuts a
request's keys 8 ways at most, which leaves most SMs idle when one request holds 100,000 keys; the
graphs for long contexts cut them as many ways as the CTAs that fit the GPU at once (measured at batch 1
and 32,768 keys: 2.83 ms per step with the 8-way graph, see the design notes for the figures after).
"""

from __future__ import annotations

from typing import Sequence

import torch

from .step import StepFunction, StepRow


LENGTH_CLASSES = (0, 8192, 32768, 131072)


def length_class(max_kv_len: int) -> int:
    return max(c for c in LENGTH_CLASSES if c <= max_kv_len)


def graph_buckets(max_bs: int) -> list[int]:
    out, b = [], 1
    while b < max_bs:
        out.append(b)
        if b >= 16 and b + b // 2 < max_bs:
            out.append(b + b // 2)
        b *= 2
    out.append(max_bs)
    return out


class _Captured:
    __slots__ = ("graph", "tokens", "logits", "f32", "i64", "launches", "sampler_scratch")

    def __init__(self, graph, tokens, logits, f32, i64, launches, sampler_scratch):
        self.graph, self.tokens, self.logits, self.f32, self.i64 = graph, tokens, logits, f32, i64
        self.launches = launches  # launches of this package's kernels inside the graph
        self.sampler_scratch = sampler_scratch  # the sampler's scratch tensor whose address the graph holds (None: none)


class DecodeGraphs:
    def __init__(self, step_fn: StepFunction, sampler, max_bs: int):
        self.step_fn = step_fn
        self.sampler = sampler
        self.buckets = graph_buckets(max_bs)
        self.max_batch = self.buckets[-1]
        cache = step_fn.cache
        # a step packs the pages its rows hold (at most the pool), one guard entry per row, and the padding rows' page
        self.indices_cap = max(g.allocator.num_blocks for g in cache.groups) + 2 * self.max_batch + 4 if cache.groups else 4
        step_fn.reserve_arena(16 * (self.max_batch + 8) + cache.num_groups * (self.indices_cap + self.max_batch + 16) + 256)
        self._generation = step_fn.arena_generation
        self._graphs: dict[tuple[int, str, int], _Captured] = {}  # (bucket, sampling mode, length class)
        self._pool = None
        self.capture_stream = torch.cuda.Stream(device=step_fn.device)
        self.replayed_launches = 0  # kernels of this package launched through graph replays so far

    def takes(self, num_rows: int) -> bool:
        return num_rows <= self.max_batch

    def _drop_all(self) -> None:
        """The arena moved: every captured address is stale. The graphs' memory pool goes with its last
        graph, so the next capture starts a new one."""
        self._graphs.clear()
        self._pool = None
        self._generation = self.step_fn.arena_generation

    def _bucket(self, n: int) -> int:
        return next(b for b in self.buckets if b >= n)

    def run(self, rows: Sequence[StepRow], sampling: dict | None, prev_tokens: torch.Tensor | None = None,
            klass: int | None = None) -> torch.Tensor:
        """One decode step (every row brings one token and wants its logits). Returns the
        sampled tokens of the real rows, int32 on the device. ``klass``: the class of context length whose
        graph to use (default: the class of the longest row; any class gives the same tokens, a graph's
        class only decides how its attention launch shares out the keys)."""
        sf = self.step_fn
        if sf.arena_generation != self._generation:
            self._drop_all()
        n = len(rows)
        bucket = self._bucket(n)
        pad = bucket - n
        mode = "greedy"
        if sampling is not None:
            mode = "top_p" if any(p < 1 for p in sampling["top_ps"]) else "temperature"
        ctx = sf.prepare(rows, pad_rows=pad, indices_cap=self.indices_cap, want_pad_rows=True, prev_tokens=prev_tokens)
        if sf.arena_generation != self._generation:  # the arena moved while preparing
            self._drop_all()
        if klass is None:
            klass = length_class(ctx.max_kv_len)
        cap = self._graphs.get((bucket, mode, klass))
        if cap is not None and cap.sampler_scratch is not None and cap.sampler_scratch is not self.sampler._scratch:
            cap = None  # the sampler has moved to a larger scratch since: the graph's address is stale
        if cap is None:
            cap = self._capture(ctx, bucket, mode, klass)
            self._graphs[(bucket, mode, klass)] = cap
        if sampling is not None:
            f32 = torch.ones((2, bucket), dtype=torch.float32)
            i64 = torch.zeros((2, bucket), dtype=torch.int64)
            f32[0, :n] = torch.tensor(sampling["temperatures"], dtype=torch.float32)
            f32[0, n:] = 0.0
            f32[1, :n] = torch.tensor(sampling["top_ps"], dtype=torch.float32)
            i64[0, :n] = torch.tensor(sampling["seeds"], dtype=torch.int64)
            i64[1, :n] = torch.tensor(sampling["counters"], dtype=torch.int64)
            cap.f32.copy_(f32.pin_memory(), non_blocking=True)
            cap.i64.copy_(i64.pin_memory(), non_blocking=True)
        cap.graph.replay()
        self.replayed_launches += cap.launches
        for r in rows:
            sf.cache.trim(r.cache)
        return cap.tokens[:n]

    def capture_all(self, modes: Sequence[str] = ("greedy",), classes: Sequence[int] = (0,)) -> int:
        """Capture the graphs of every batch bucket now instead of at their first use (the reference
        captures at start-up, miniserve/engine/cuda_graph.py), for the given classes of context length.
        Needs an idle cache: it steps ``max_batch`` one-token requests that it creates and releases.
        Returns how many it captured."""
        sf = self.step_fn
        sampling_for = {
            "greedy": lambda n: None,
            "temperature": lambda n: dict(temperatures=[1.0] * n, top_ps=[1.0] * n, seeds=[0] * n, counters=[0] * n),
            "top_p": lambda n: dict(temperatures=[1.0] * n, top_ps=[0.5] * n, seeds=[0] * n, counters=[0] * n),
        }
        before = len(self._graphs)
        for mode, klass in ((m, k) for m in modes for k in classes):
            for bucket in self.buckets:
                caches = [sf.cache.new_request() for _ in range(bucket)]
                try:
                    self.run([StepRow(c, [0], (0,)) for c in caches], sampling_for[mode](bucket), klass=klass)
                finally:
                    for c in caches:
                        sf.cache.release(c)
        torch.cuda.current_stream(sf.device).synchronize()
        return len(self._graphs) - before

    def _forward(self, ctx, bucket: int, mode: str, klass: int, f32, i64):
        sf = self.step_fn
        ctx.stream = torch.cuda.current_stream(sf.device).cuda_stream
        ctx.graph_bucket = bucket
        ctx.graph_kv_len = klass
        logits = sf.model.forward(ctx, sf.cache.entry_views)
        tokens = torch.empty(bucket, dtype=torch.int32, device=sf.device)
        from .. import ops

        if mode == "greedy":
            ops.sample(tokens, logits, stream=ctx.stream)
        else:
            ops.sample(tokens, logits, temperature=f32[0], top_p=f32[1] if mode == "top_p" else None, seed=i64[0],
                       counter=i64[1], scratch=self.sampler._scratch if mode == "top_p" else None,
                       stream=ctx.stream)
        return logits, tokens

    def _capture(self, ctx, bucket: int, mode: str, klass: int) -> _Captured:
        sf = self.step_fn
        f32 = torch.zeros((2, bucket), dtype=torch.float32, device=sf.device)
        f32[1] = 1.0
        i64 = torch.zeros((2, bucket), dtype=torch.int64, device=sf.device)
        self.sampler._ensure(bucket)
        torch.cuda.current_stream(sf.device).synchronize()
        s = self.capture_stream
        # A warm-up pass outside the capture (first-use set-up of kernels and libraries must not happen while
        # capturing). It runs the step's real rows, so what it changes has to be put back: rewriting the same
        # keys and values is harmless, but a mixer's per-request state would otherwise advance twice (by the
        # warm-up and again by the first replay).
        from ..cache.manager import StateEntryView

        slots = ctx.state_slot.long()
        states = {id(v.state): v.state for v in sf.cache.entry_views if isinstance(v, StateEntryView) and v.state is not None}
        kept = [(st, st[slots].clone()) for st in states.values()]
        with torch.cuda.stream(s):
            s.wait_stream(torch.cuda.current_stream(sf.device))
            self._forward(ctx, bucket, mode, klass, f32, i64)
        s.synchronize()
        for st, value in kept:
            st[slots] = value
        torch.cuda.current_stream(sf.device).synchronize()
        from ..ops import native

        import gc

        graph = torch.cuda.CUDAGraph()
        before = native.LAUNCHES[0]
        collecting = gc.isenabled()  # no collection while the capture is open (see StepGraphs._capture)
        try:
            with torch.cuda.graph(graph, pool=self._pool, stream=s):
                gc.disable()
                logits, tokens = self._forward(ctx, bucket, mode, klass, f32, i64)
        finally:
            if collecting:
                gc.enable()
        launches = native.LAUNCHES[0] - before
        native.LAUNCHES[0] = before  # a capture launches nothing
        if self._pool is None:
            self._pool = graph.pool()
        return _Captured(graph, tokens, logits, f32, i64, launches, self.sampler._scratch if mode == "top_p" else None)


class _Recorder:
    """Captures one pass of the model as a chain of pieces: CUDA graphs, and between them the calls
    that operations kept out of the graphs (``defer``)."""

    def __init__(self, pool, stream: torch.cuda.Stream, single_rows: int, lasting: dict):
        self.pool, self.stream = pool, stream
        self.lasting = lasting  # what captures of different shapes share (scratch that only one step at a time uses)
        self.pieces: list = []  # torch.cuda.CUDAGraph | callable(ctx)
        self.hooks: list = []  # callable(ctx), run before the pieces of every replay
        self.shared: dict = {}  # what operations of one captured pass share (a plan written once per step, say)
        # how many rows at the front of every step of the captured shape bring a single token (decoding
        # rows, which attention sends to another kernel than the rest)
        self.single_rows = single_rows
        self._open: torch.cuda.CUDAGraph | None = None

    def begin(self) -> None:
        self._open = torch.cuda.CUDAGraph()
        self._open.capture_begin(pool=self.pool)

    def end(self) -> None:
        if self._open is not None:
            self._open.capture_end()
            self.pieces.append(self._open)
            self._open = None

    def defer(self, call) -> None:
        """Keep ``call(ctx)`` out of the graphs: it is made between them, with every step's own context."""
        self.end()
        self.pieces.append(call)
        self.begin()

    def before(self, call) -> None:
        """Have ``call(ctx)`` made before the graphs of every step that replays them (and of this one)."""
        self.hooks.append(call)


class _Pieces:
    __slots__ = ("pieces", "hooks", "logits", "layout", "launches", "uses")

    def __init__(self, pieces, hooks, logits, layout, launches):
        self.pieces, self.hooks, self.logits, self.layout, self.launches, self.uses = pieces, hooks, logits, layout, launches, 0


class StepGraphs:
    """Prompt and mixed steps of a shape that comes again, replayed from CUDA graphs.

    A step that is not decode-only launches a couple of hundred kernels from Python; for a small model
    the stream launches cost more than the host takes to issue them (Qwen3-0.6B sizes, 2,048 tokens:
    3.86 ms launched eagerly with the host ahead, 3.59 ms replayed). What the kernels of such a step
    get from the host is the number of tokens, of rows and of wanted logits; everything else they read
    from the step's arrays, which the packer lays out at fixed places for a given (tokens, rows,
    wanted) when it is given a fixed number of page entries. The exception is attention, whose
    kernels, grids and key splits follow the rows' lengths and starts. With head size 128 the decoding
    rows at the front of a step (their number is part of the shape) go to the split-key kernel as
    inside a decode graph, and the tcgen05 kernel for the rest is launched with a CTA per SM and reads
    its plan from device memory, where a hook writes it before every replay: the step is one graph.
    Else ``ops.attention`` keeps itself out of the capture and is called again for every step, between
    the graphs.

    Shapes come again more often when the number of tokens is rounded up: a step is padded with one row
    of its own (tokens that write to the page outside the allocator and whose results nobody reads) to
    the next multiple of 32 tokens up to 256, of 64 up to 512, of 128 beyond, so that a prompt of any
    length meets one of two dozen shapes (a lone prompt of 128 tokens at Qwen3-0.6B sizes: 3.7 ms
    launched from Python, of which the device is busy for one). In float32 the real rows' results do not
    depend on the padding; in bfloat16 the products of the padded step may round differently, within
    what another cut of the same tokens would change.

    A step whose (tokens, rows, wanted, decoding rows) have been seen ``sightings`` times is captured while
    it runs, later ones replay; a step without decoding rows (prompts alone) at its second sighting, and
    with an eighth of the distance that is otherwise kept between two captures. Only models whose parts all declare ``shape_static`` are taken. The least recently used shapes are
    dropped beyond ``max_shapes``. The logits of a replayed step live in the graphs' memory and are
    overwritten by the next replayed step.
    """

    def __init__(self, step_fn: StepFunction, indices_cap: int, max_shapes: int = 32, min_tokens: int = 16,
                 max_step_flops: float = 8e12, capture_every: int = 64, sightings: int = 4, pad: bool = True):
        self.step_fn = step_fn
        self.pad = pad
        self.indices_cap = indices_cap
        self.max_shapes, self.min_tokens = max_shapes, min_tokens
        self.enabled = bool(step_fn.model.shape_static)
        # Only steps that the launches weigh on are taken: a step of more than max_step_flops (about 6 ms of
        # products at the tensor cores' rate) gains nothing measurable from a replay, and its capture is
        # a whole pass of the host over a large model (Qwen3-8B sizes, 32 requests with prompts of 128 to
        # 4,096 tokens: the 2,048-token steps took 36 ms on average with their shapes captured at the
        # second sighting, 31 ms without).
        model = step_fn.model
        per_weight = 2 if model.dtype == torch.bfloat16 else 4
        self.flops_per_token = 2.0 * model.weight_bytes() / per_weight if model.bound else 0.0
        self.max_step_flops = max_step_flops
        # A capture costs the host about 6 ms (Qwen3-0.6B sizes), during which steps already launched go
        # on; a replay saves the device 0.3 ms of a 2,048-token step and the host most of its 2.6 ms of
        # launching, which counts where steps are short (a 256-token step: 3.8 -> 2.0 ms). Loads whose
        # shapes keep changing gain nothing from captures, so they are kept rare: a shape is captured at
        # its fourth sighting, at most one in `capture_every` steps that the graphs are asked about.
        # Measured with 128 to 256 requests of random lengths (tools/stress): within 1 % either way of
        # the same run without these graphs; the same step again and again (bench.py's prefill) 4.14 -> 3.46 ms
        # together with the kernels' gains.
        self.capture_every, self.sightings = capture_every, sightings
        self._since_capture = capture_every
        self._lasting: dict = {}
        self._seen: dict[tuple, int] = {}
        self._shapes: dict[tuple, _Pieces] = {}  # insertion order = least recently used first
        self._pool = None
        self._generation = step_fn.arena_generation
        self.capture_stream = torch.cuda.Stream(device=step_fn.device)
        self.replayed_launches = 0  # kernels of this package launched from inside replayed graphs
        self.captures = 0

    def _drop_all(self) -> None:
        """The arena moved: every captured address is stale. The graphs' memory pool goes with its last
        graph, so the next capture starts a new one."""
        self._shapes.clear()
        self._lasting.clear()
        self._pool = None
        self._generation = self.step_fn.arena_generation

    @staticmethod
    def padded(tokens: int) -> int:
        """The number of tokens that a step of ``tokens`` is run with."""
        unit = 32 if tokens <= 256 else 64 if tokens <= 512 else 128
        return -(-tokens // unit) * unit

    def _key(self, rows: Sequence[StepRow]) -> tuple | None:
        tokens = sum(len(r.tokens) for r in rows)
        if not self.enabled or tokens < self.min_tokens or tokens == len(rows):  # decode-only steps have graphs of their own
            return None
        run_with = self.padded(tokens) if self.pad else tokens
        if run_with * self.flops_per_token > self.max_step_flops:
            return None
        # decoding rows come first in a mixed step; how many there are decides which attention kernels run on what
        single = next((i for i, r in enumerate(rows) if len(r.tokens) != 1), len(rows))
        # (tokens run, rows with the padding row, wanted logits, decoding rows at the front)
        return run_with, len(rows) + (run_with != tokens), sum(len(r.want) for r in rows), single

    def run(self, rows: Sequence[StepRow], prev_tokens: torch.Tensor | None = None) -> torch.Tensor | None:
        """The step's logits, or None if this step is left to the eager path (nothing was touched then)."""
        key = self._key(rows)
        if key is None:
            return None
        sf = self.step_fn
        if sf.arena_generation != self._generation:
            self._drop_all()
        held = self._shapes.get(key)
        self._since_capture += 1
        if held is None:
            n = self._seen.get(key, 0) + 1
            if len(self._seen) > 4096:
                self._seen.clear()
            self._seen[key] = n
            # prompts alone come in few shapes once padded, and come again: they are captured sooner
            sightings, gap = (self.sightings, self.capture_every) if key[3] else (min(self.sightings, 2), self.capture_every // 8)
            if n < sightings or self._since_capture <= gap:
                return None
        pad = key[0] - sum(len(r.tokens) for r in rows)
        ctx = sf.prepare(rows, pad_rows=1 if pad else 0, pad_len=max(pad, 1), indices_cap=self.indices_cap, prev_tokens=prev_tokens)
        if sf.arena_generation != self._generation:  # it moved while preparing this step
            self._drop_all()
            held = None
        if held is not None and held.layout != ctx.layout:
            held = None  # cannot happen for one key; checked because a graph that reads the wrong place reads garbage silently
        if held is None:
            held = self._capture(ctx, single_rows=key[3])
            self._shapes.pop(key, None)
            self._shapes[key] = held
            self._since_capture = 0
            while len(self._shapes) > self.max_shapes:
                dropped = next(iter(self._shapes))
                self._shapes.pop(dropped)
                self._seen.pop(dropped, None)  # it has to come twice again
        else:
            self._shapes[key] = self._shapes.pop(key)  # now the most recently used
        ctx.stream = torch.cuda.current_stream(sf.device).cuda_stream
        for hook in held.hooks:
            hook(ctx)
        for piece in held.pieces:
            if isinstance(piece, torch.cuda.CUDAGraph):
                piece.replay()
            else:
                piece(ctx)
        held.uses += 1
        self.replayed_launches += held.launches
        return held.logits

    def capture_prompt_shapes(self, max_tokens: int) -> int:
        """Capture now, on an idle cache, the shapes that lone prompts of up to ``max_tokens`` tokens meet
        (every padded size up to there), instead of at their second sighting: each size is first run
        once as it is (what a kernel or the library sets up at its first use must not happen inside a
        capture), then captured from a prompt one token shorter. Returns how many were captured."""
        if not self.enabled or not self.pad:
            return 0
        sf = self.step_fn
        sizes = sorted({self.padded(n) for n in range(max(self.min_tokens, 2), max_tokens + 1)})
        room = min((g.allocator.num_blocks for g in sf.cache.groups), default=0) * sf.cache.page_size if sf.cache.groups else max_tokens
        sizes = [n for n in sizes if n <= min(max_tokens, room) and n * self.flops_per_token <= self.max_step_flops]
        before = self.captures
        kept = self.sightings, self.capture_every, self.max_shapes
        self.max_shapes = max(self.max_shapes, len(self._shapes) + len(sizes))
        try:
            for n in sizes:
                for tokens, sightings in ((n, 1 << 30), (n - 1, 1)):
                    rows = [StepRow(sf.cache.new_request(), [0] * tokens, (tokens - 1,))]
                    self.sightings, self.capture_every, self._since_capture = sightings, 0, 1
                    try:
                        if self._key(rows) not in self._shapes:
                            sf.run(rows)
                    finally:
                        sf.cache.release(rows[0].cache)
        finally:
            self.sightings, self.capture_every = kept[0], kept[1]
        torch.cuda.current_stream(sf.device).synchronize()
        return self.captures - before

    def _capture(self, ctx, single_rows: int) -> _Pieces:
        from ..ops import native

        import gc

        sf = self.step_fn
        # (no wait for the device: a capture launches nothing, and steps still running go on meanwhile)
        if self._pool is None:
            self._pool = torch.cuda.graph_pool_handle()
        s = self.capture_stream
        rec = _Recorder(self._pool, s, single_rows, self._lasting)
        before = native.LAUNCHES[0]
        ctx.recorder = rec
        # No garbage collection while a capture is open: a graph of an earlier, dropped set that the
        # collector frees in the middle of it destroys its CUDA objects, which is not allowed then and
        # voids the capture. What is garbage already goes now.
        gc.collect()
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.stream(s):
                ctx.stream = s.cuda_stream
                rec.begin()
                try:
                    logits = sf.model.forward(ctx, sf.cache.entry_views)
                finally:
                    rec.end()
        finally:
            ctx.recorder = None
            if collecting:
                gc.enable()
        launches = native.LAUNCHES[0] - before
        native.LAUNCHES[0] = before  # a capture launches nothing
        self.captures += 1
        return _Pieces(rec.pieces, rec.hooks, logits, ctx.layout, launches)
