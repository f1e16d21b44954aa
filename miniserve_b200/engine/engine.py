"""The engine loop: step() = schedule -> launch (step function + sampling, nothing waits for the
device) -> read back the PREVIOUS step's tokens and finish what ended.

The same loop as miniserve/engine/engine.py:137-204. With overlap scheduling (the default) a step
is launched before the previous one is read back, so the host schedules and packs step t+1 while
the GPU still runs step t:

* a request that sampled a token in step t gets a placeholder output token, and its input id in
  step t+1 is taken from step t's sampled tokens on the device;
* a request that has sampled its last allowed token is not scheduled again;
* a request that turns out to have sampled a stop token in step t was already given a row in
  step t+1; that token is dropped when step t+1 is read back.

Giving back the pages of a request that ended in step t while step t+1 still uses them is safe:
they can be handed out again only when step t+2 is formed, and that runs after t+1 on the same
stream.
"""

from __future__ import annotations

import itertools
import random
from typing import Sequence

import torch

from ..cache.manager import CacheManager, group_needs, window_pages
from ..parts.decoder import DecoderModel
from ..sampling.sampler import Sampler
from .request import PLACEHOLDER, Request, RequestState, SamplingParams
from .scheduler import Plan, Scheduler
from .step import StepError, StepFunction, StepRow

DEFAULT_CHUNKED_PREFILL = 2048


def _numel(shape) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


class _range:
    """An NVTX range around a phase of a step when ``MINISERVE_NVTX=1`` (a profiler's timeline then shows
    schedule / launch / read back per step, as miniserve/bench/offline.py:235-241 brackets its steps);
    nothing otherwise."""

    enabled = __import__("os").environ.get("MINISERVE_NVTX", "0") == "1"

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if self.enabled:
            torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        if self.enabled:
            torch.cuda.nvtx.range_pop()
        return False


class _Launched:
    """A launched step: its plan, the sampled tokens on the device (one per sampling row, then the
    kernels' status word), their host copy once ``done``, each request's row among the sampled
    tokens, and each sampling row's request and output slot."""

    __slots__ = ("plan", "tokens", "host", "done", "row_of", "slots")

    def __init__(self, plan, tokens, host, done, row_of, slots):
        self.plan, self.tokens, self.host, self.done, self.row_of, self.slots = plan, tokens, host, done, row_of, slots


class Engine:
    def __init__(self, model: DecoderModel, kv_pool_tokens: int | None = None, page_size: int = 16,
                 max_running: int = 64, max_prefill_tokens: int = 8192, chunked_prefill_size: int | None = None,
                 seed: int = 0, cuda_graph: bool = True, cuda_graph_max_bs: int | None = None,
                 kv_mem_fraction: float = 0.9, overlap: bool = True, cache: CacheManager | None = None, step_fn=None,
                 sampler=None, poison_on_free: bool = False, step_graphs: bool = True, schedule_policy: str = "fcfs"):
        """``kv_pool_tokens``: exact size of the cache pool in tokens, rounded down to whole pages
        (default: ``kv_mem_fraction`` of the memory the device has free after the weights, less a
        reserve for activations). ``chunked_prefill_size``: tokens per step, decode tokens included,
        with prompts cut into portions and batched with decode tokens; 0 keeps whole prompts in
        prefill-only steps; default 2048. ``seed`` seeds the sampling of requests that bring no
        seed of their own, in submission order. ``cuda_graph``: replay captured CUDA graphs for
        decode-only steps of up to ``cuda_graph_max_bs`` requests (default ``max_running``).
        ``step_graphs``: with ``cuda_graph``, also capture prompt and mixed steps whose shape comes again.
        ``overlap``: launch each step before reading back the previous one.
        ``schedule_policy``: "fcfs" or "sjf" (``Scheduler``).
        Names and meanings follow miniserve/engine/engine.py:42-77. ``cache``, ``step_fn`` and
        ``sampler`` replace the ones the engine would build (a test can run the whole loop on the
        host against a stand-in step function this way). ``poison_on_free``: a debugging aid, see
        ``CacheManager``."""
        self.model = model
        if chunked_prefill_size is None:
            chunked_prefill_size = DEFAULT_CHUNKED_PREFILL
        step_tokens = chunked_prefill_size if chunked_prefill_size else max_prefill_tokens
        if cache is None:
            num_pages = self._pool_pages(model, kv_pool_tokens, page_size, kv_mem_fraction, step_tokens, max_running)
            cache = CacheManager(model.entry_caches, num_pages, page_size, max_running, dtype=model.dtype,
                                 device=model.device, poison_on_free=poison_on_free, step_tokens=step_tokens)
        self.cache = cache
        self.settings = dict(kv_pool_tokens=kv_pool_tokens, page_size=page_size, max_running=max_running,
                             max_prefill_tokens=max_prefill_tokens, chunked_prefill_size=chunked_prefill_size, seed=seed,
                             cuda_graph=cuda_graph, cuda_graph_max_bs=cuda_graph_max_bs or max_running, overlap=overlap,
                             schedule_policy=schedule_policy)
        self.step_fn = step_fn if step_fn is not None else StepFunction(model, self.cache)
        self.scheduler = Scheduler(self.cache, max_running, max_prefill_tokens, chunked_prefill_size, schedule_policy)
        self.sampler = sampler if sampler is not None else Sampler(model.device, model.spec.vocab_size, max_running)
        self.requests: dict[int, Request] = {}
        self._rids = itertools.count()
        self._seeds = random.Random(seed)
        self.logits_hook = None  # called with (plan, logits) before sampling; for diagnostics
        self.graphs = None
        if cuda_graph and step_fn is None:
            from .graphs import DecodeGraphs

            self.graphs = DecodeGraphs(self.step_fn, self.sampler, cuda_graph_max_bs or max_running)
            if step_graphs and model.shape_static:
                from .graphs import StepGraphs

                # the arena holds the largest step at the fixed layout now, so that it does not move under captured graphs
                budget = (chunked_prefill_size if chunked_prefill_size else max_prefill_tokens) + max_running
                # (a padded step's extra row brings up to 128 tokens and their page entries)
                cap = self.graphs.indices_cap + -(-128 // self.cache.page_size)
                self.step_fn.reserve_arena(3 * (budget + 132) + 6 * (max_running + 8)
                                           + self.cache.num_groups * (cap + max_running + 16) + 256)
                self.step_fn.graphs = StepGraphs(self.step_fn, cap)
        self.overlap = overlap
        self.num_steps = 0
        self.stalled = False  # the last step() neither launched a step nor read one back
        self.launched: Plan | None = None  # the plan the last step() launched
        self._inflight: _Launched | None = None
        self._pinned: list[torch.Tensor] = []

    @staticmethod
    def _pool_pages(model, kv_pool_tokens, page_size, fraction, step_tokens, max_running) -> list[int]:
        """Pages for each cache group (in ``group_needs`` order). A group that keeps every key gets
        ``kv_pool_tokens`` worth of pages, or its share of the device memory that is left after the
        weights, the per-request state tensors and a reserve for a step's activations; a windowed
        group never needs more than ``max_running`` requests' windows, and gets no more."""
        item = torch.empty((), dtype=model.dtype).element_size()
        needs, states = group_needs(model.entry_caches)
        page_bytes = [2 * count * need.kv_heads * need.head_dim * item * page_size for need, count in needs]
        bound = [max_running * window_pages(need.window, page_size, step_tokens) if need.window else None for need, _ in needs]
        if kv_pool_tokens is not None:
            if kv_pool_tokens < page_size:
                raise ValueError(f"kv_pool_tokens={kv_pool_tokens} is smaller than one page ({page_size})")
            want = kv_pool_tokens // page_size
            return [want if b is None else min(want, b) for b in bound]
        free, _ = torch.cuda.mem_get_info(model.device)
        state_bytes = sum(max_running * torch.empty((), dtype=st.dtype).element_size() * _numel(st.shape) for st in states)
        # activations of the largest step: a few [tokens, widest] buffers, and float32 logits of every row
        widest = max(model.spec.hidden_size * 8, 1)
        reserve = step_tokens * widest * 4 * 4 + max_running * model.spec.vocab_size * 4 * 3 + (1 << 30)
        usable = int(fraction * (free - reserve - state_bytes))
        windowed = sum(b * pb for b, pb in zip(bound, page_bytes) if b is not None)
        whole = sum(pb for b, pb in zip(bound, page_bytes) if b is None)
        pages = (usable - windowed) // max(whole, 1) if whole else 0
        if usable <= windowed or (whole and pages < 1):
            raise RuntimeError(f"no device memory left for the cache pool ({free} bytes free)")
        return [pages if b is None else b for b in bound]

    def describe(self) -> dict:
        """The configuration in effect, as plain data (what a benchmark records beside its numbers;
        miniserve/engine/describe.py:22-44 serves the same purpose)."""
        m, c = self.model, self.cache
        return dict(
            architecture=m.spec.architecture, dtype=str(m.dtype).replace("torch.", ""), device=str(m.device),
            layers=len(m.spec.run_order), hidden_size=m.spec.hidden_size, vocab_size=m.spec.vocab_size,
            weight_bytes=m.weight_bytes() if m.bound else None,
            cache_groups=[dict(entries=len(g.entries), kv_heads=g.need.kv_heads, head_dim=g.need.head_dim, window=g.need.window,
                               pages=g.allocator.num_blocks, page_size=g.page_size) for g in c.groups],
            cache_bytes=c.pool_bytes(), cache_bytes_per_token=c.bytes_per_token(), state_bytes=c.state_bytes(),
            request_slots=c.max_requests, graph_buckets=list(self.graphs.buckets) if self.graphs is not None else [],
            step_graphs=getattr(self.step_fn, "graphs", None) is not None, **self.settings)

    # ------------------------------------------------------------------ requests
    def capture_graphs(self, modes=("greedy",), context_lengths=(0,), prompt_tokens: int = 0) -> int:
        """Capture the decode graphs of every batch bucket now (while the engine is idle) instead
        of at their first use; returns how many were captured. ``modes``: of "greedy",
        "temperature", "top_p". ``context_lengths``: lengths that requests will reach; the graphs of
        every class of context length from the shortest's to the longest's are captured (those for short
        contexts by default). ``prompt_tokens``: also capture the step graphs that lone prompts of up to so
        many tokens meet (no more than a step's token budget), so that the first requests replay them."""
        if self.graphs is None:
            return 0
        if self.has_unfinished:
            raise RuntimeError("graphs are captured at the start, before any request is submitted")
        from .graphs import LENGTH_CLASSES, length_class

        lo, hi = (length_class(max(int(f(context_lengths)), 1)) for f in (min, max))
        count = self.graphs.capture_all(modes, [c for c in LENGTH_CLASSES if lo <= c <= hi])
        step_graphs = getattr(self.step_fn, "graphs", None)
        if prompt_tokens and step_graphs is not None:
            count += step_graphs.capture_prompt_shapes(min(prompt_tokens, self.scheduler.chunked_prefill_size or prompt_tokens))
        return count

    def add_request(self, prompt_ids: Sequence[int], params: SamplingParams) -> Request:
        req = Request(next(self._rids), list(prompt_ids), params)
        req.seed = params.seed if params.seed is not None else self._seeds.randrange(2 ** 32)
        self.scheduler.add(req)
        self.requests[req.rid] = req
        return req

    def abort(self, rid: int) -> None:
        req = self.requests.get(rid)
        if req is None:
            return
        req.transition(RequestState.ABORTED)
        self._retire(req)

    @property
    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished or self._inflight is not None

    def _retire(self, req: Request) -> None:
        req.drop_pending()
        if req.cache is not None:
            self.cache.release(req.cache)
            req.cache = None
        self.scheduler.retire(req)
        del self.requests[req.rid]

    # ------------------------------------------------------------------ the loop
    def step(self) -> Plan | None:
        """Run one step. Returns the plan launched by this call (None if nothing could run). With
        overlap the tokens it samples are read back by the NEXT call."""
        with _range("schedule"):
            plan = self.scheduler.schedule()
        prev = self._inflight
        self.launched = plan
        with _range(f"launch {plan.phase} rows={len(plan.rows)} tokens={plan.num_tokens}" if plan is not None else "launch none"):
            self._inflight = self._launch(plan, prev) if plan is not None else None
        if not self.overlap:
            prev, self._inflight = self._inflight, None
        if prev is not None:
            with _range("read back"):
                self._process(prev)
        # a step that neither launched nor read anything back changed nothing: the next would do the same
        self.stalled = plan is None and prev is None
        return plan

    def _launch(self, plan: Plan, prev: _Launched | None) -> _Launched:
        self.num_steps += 1
        sampling = [r for r in plan.rows if r.completes]
        reqs = [r.request for r in sampling]
        greedy = all(r.params.is_greedy for r in reqs)
        args = None if greedy else dict(
            temperatures=[r.params.temperature for r in reqs], top_ps=[r.params.top_p for r in reqs],
            seeds=[r.seed for r in reqs], counters=[r.seq_len for r in reqs])
        rows = []
        prev_tokens = None
        for r in plan.rows:
            req = r.request
            tokens = req.token_slice(r.start, r.count)
            fill_from = None
            if tokens and tokens[-1] == PLACEHOLDER:
                # only a decode row's single input can be a token that is not read back yet
                if r.count != 1 or prev is None or req.rid not in prev.row_of:
                    raise RuntimeError("a placeholder token outside a decode row, or without the step that sampled it")
                fill_from, prev_tokens, tokens = prev.row_of[req.rid], prev.tokens, [0]
            rows.append(StepRow(req.cache, tokens, (r.count - 1,) if r.completes else (), fill_from))
        if self.graphs is not None and self.logits_hook is None and plan.phase == "decode" and self.graphs.takes(len(rows)):
            tokens = self.graphs.run(rows, args, prev_tokens=prev_tokens)
        else:
            logits = self.step_fn.run(rows, prev_tokens=prev_tokens) if prev_tokens is not None else self.step_fn.run(rows)
            if self.logits_hook is not None:
                self.logits_hook(plan, logits)
            tokens = self.sampler.sample(logits, **(args or {}))
        n = len(reqs)
        both = torch.cat((tokens[:n], self.step_fn.status))
        host, done = both, None
        if both.is_cuda:
            host = self._pinned_buffer(n + 1)
            host.copy_(both, non_blocking=True)
            done = torch.cuda.Event()
            done.record()
        slots = []
        for req in reqs:
            slots.append((req, len(req.output_ids)))
            req.output_ids.append(PLACEHOLDER)
            req.num_pending += 1
            if req.state is RequestState.PREFILL:
                req.transition(RequestState.DECODE)
        return _Launched(plan, tokens, host, done, {req.rid: i for i, req in enumerate(reqs)}, slots)

    def _pinned_buffer(self, n: int) -> torch.Tensor:
        """Two pinned staging buffers in turn: the one a launch writes was read back a step ago."""
        if len(self._pinned) < 2 or self._pinned[0].numel() < n:
            size = max(n, 2 * (self._pinned[0].numel() if self._pinned else 64))
            self._pinned = [torch.empty(size, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._pinned.reverse()
        return self._pinned[0][:n]

    def _process(self, launched: _Launched) -> None:
        """Wait for the launched step's tokens (the one device-to-host wait of a step), put them in
        place of the placeholders, and retire the requests that ended."""
        if launched.done is not None:
            launched.done.synchronize()
        values = launched.host.tolist()
        status = values.pop()
        if status:
            # the step after this one is already launched: let it drain, then put the status word and the
            # kernels' tickets back to zero (as StepFunction.check_status does), so that a caller who
            # catches the error can go on
            self.step_fn.reset_after_fault()
            raise StepError(f"a kernel reported a fault it caught itself (code {status})")
        for (req, slot), tok in zip(launched.slots, values):
            if req.is_done:  # ended before (this token lies past its end)
                continue
            req.output_ids[slot] = tok
            req.num_pending -= 1
            if slot + 1 >= req.params.max_new_tokens or tok in req.params.stop_token_ids:
                req.drop_pending()
                req.transition(RequestState.FINISHED)
                self._retire(req)

    def generate(self, prompts: Sequence[Sequence[int]], params: SamplingParams | Sequence[SamplingParams],
                 on_step=None, max_steps: int | None = None) -> list[list[int]]:
        """Submit all prompts (token ids) at once and run to completion; output token ids per prompt.
        ``on_step(engine, plan)`` is called after every step with the plan that step launched (None if it
        launched nothing): a place to count, time or check. ``max_steps``: raise if not done by then."""
        if isinstance(params, SamplingParams):
            params = [params] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError(f"{len(prompts)} prompts but {len(params)} sampling parameters")
        reqs: list[Request] = []
        try:
            for p, sp in zip(prompts, params):
                reqs.append(self.add_request(p, sp))
        except Exception:
            # a prompt was refused: none of this call's requests stays behind in the queues
            for r in reqs:
                self.abort(r.rid)
            raise
        steps = 0
        while self.has_unfinished:
            if max_steps is not None and steps >= max_steps:
                raise RuntimeError(f"not finished after {steps} steps")
            plan = self.step()
            steps += 1
            # (a step may launch nothing and still move on: with overlap, a preempted request waits for its
            # newest token to be read back before it is admitted again, and this step read it)
            if self.stalled and self.scheduler.has_unfinished:
                raise RuntimeError("the scheduler produced no step although requests are unfinished")
            if on_step is not None:
                on_step(self, plan)
        return [r.output_ids for r in reqs]
