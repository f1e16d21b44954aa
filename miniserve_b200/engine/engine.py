"""The engine loop: step() = schedule -> step function -> sample -> read back -> finish.

The same loop as miniserve/engine/engine.py:137-204 without its one-step-lag overlap: each step
reads its sampled tokens back before the next is scheduled. Sampling stays on the device; the
host reads the tokens (and the kernels' status word) once per step.
"""

from __future__ import annotations

import itertools
import random
from typing import Sequence

import torch

from ..cache.manager import CacheManager
from ..parts.decoder import DecoderModel
from ..sampling.sampler import Sampler
from .request import Request, RequestState, SamplingParams
from .scheduler import Plan, Scheduler
from .step import StepError, StepFunction, StepRow

DEFAULT_CHUNKED_PREFILL = 2048


class Engine:
    def __init__(self, model: DecoderModel, kv_pool_tokens: int | None = None, page_size: int = 16,
                 max_running: int = 64, max_prefill_tokens: int = 8192, chunked_prefill_size: int | None = None,
                 seed: int = 0, cuda_graph: bool = True, cuda_graph_max_bs: int | None = None,
                 kv_mem_fraction: float = 0.9, cache: CacheManager | None = None, step_fn=None, sampler=None):
        """``kv_pool_tokens``: exact size of the cache pool in tokens, rounded down to whole pages
        (default: ``kv_mem_fraction`` of the memory the device has free after the weights, less a
        reserve for activations). ``chunked_prefill_size``: tokens per step, decode tokens included,
        with prompts cut into portions and batched with decode tokens; 0 keeps whole prompts in
        prefill-only steps; default 2048. ``seed`` seeds the sampling of requests that bring no
        seed of their own, in submission order. ``cuda_graph``: replay captured CUDA graphs for
        decode-only steps of up to ``cuda_graph_max_bs`` requests (default ``max_running``).
        Names and meanings follow miniserve/engine/engine.py:42-77. ``cache``, ``step_fn`` and
        ``sampler`` replace the ones the engine would build (a test can run the whole loop on the
        host against a stand-in step function this way)."""
        self.model = model
        if chunked_prefill_size is None:
            chunked_prefill_size = DEFAULT_CHUNKED_PREFILL
        if cache is None:
            num_pages = self._pool_pages(model, kv_pool_tokens, page_size, kv_mem_fraction,
                                         chunked_prefill_size if chunked_prefill_size else max_prefill_tokens,
                                         max_running)
            cache = CacheManager(model.entry_caches, num_pages, page_size, max_running, dtype=model.dtype,
                                 device=model.device)
        self.cache = cache
        self.step_fn = step_fn if step_fn is not None else StepFunction(model, self.cache)
        self.scheduler = Scheduler(self.cache, max_running, max_prefill_tokens, chunked_prefill_size)
        self.sampler = sampler if sampler is not None else Sampler(model.device, model.spec.vocab_size, max_running)
        self.requests: dict[int, Request] = {}
        self._rids = itertools.count()
        self._seeds = random.Random(seed)
        self.logits_hook = None  # called with (plan, logits) before sampling; for diagnostics
        self.graphs = None
        if cuda_graph and step_fn is None:
            from .graphs import DecodeGraphs

            self.graphs = DecodeGraphs(self.step_fn, self.sampler, cuda_graph_max_bs or max_running)
        self.num_steps = 0

    @staticmethod
    def _pool_pages(model, kv_pool_tokens, page_size, fraction, step_tokens, max_running) -> int:
        per_token = 0
        item = torch.empty((), dtype=model.dtype).element_size()
        seen = set()
        for ec in model.entry_caches:
            if ec.need is not None and ec.owner not in seen and hasattr(ec.need, "kv_heads"):
                seen.add(ec.owner)
                per_token += 2 * ec.need.kv_heads * ec.need.head_dim * item
        if kv_pool_tokens is not None:
            if kv_pool_tokens < page_size:
                raise ValueError(f"kv_pool_tokens={kv_pool_tokens} is smaller than one page ({page_size})")
            return kv_pool_tokens // page_size
        free, _ = torch.cuda.mem_get_info(model.device)
        # activations of the largest step: a few [tokens, widest] buffers, and float32 logits of every row
        widest = max(model.spec.hidden_size * 8, 1)
        reserve = step_tokens * widest * 4 * 4 + max_running * model.spec.vocab_size * 4 * 3 + (1 << 30)
        usable = int(fraction * (free - reserve))
        pages = usable // max(per_token * page_size, 1)
        if pages < 1:
            raise RuntimeError(f"no device memory left for the cache pool ({free} bytes free)")
        return pages

    # ------------------------------------------------------------------ requests
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
        return self.scheduler.has_unfinished

    def _retire(self, req: Request) -> None:
        if req.cache is not None:
            self.cache.release(req.cache)
            req.cache = None
        self.scheduler.retire(req)
        del self.requests[req.rid]

    # ------------------------------------------------------------------ the loop
    def step(self) -> Plan | None:
        plan = self.scheduler.schedule()
        if plan is None:
            return None
        self.num_steps += 1
        sampling = [r for r in plan.rows if r.completes]
        reqs = [r.request for r in sampling]
        greedy = all(r.params.is_greedy for r in reqs)
        args = None if greedy else dict(
            temperatures=[r.params.temperature for r in reqs], top_ps=[r.params.top_p for r in reqs],
            seeds=[r.seed for r in reqs], counters=[r.seq_len for r in reqs])
        rows = [StepRow(r.request.cache, r.request.token_slice(r.start, r.count),
                        (r.count - 1,) if r.completes else ()) for r in plan.rows]
        if self.graphs is not None and self.logits_hook is None and plan.phase == "decode" and self.graphs.takes(len(rows)):
            tokens = self.graphs.run(rows, args)
        else:
            logits = self.step_fn.run(rows)
            if self.logits_hook is not None:
                self.logits_hook(plan, logits)
            tokens = self.sampler.sample(logits, **(args or {}))
        host = torch.cat((tokens[:len(reqs)], self.step_fn.status)).tolist()
        if host[-1]:
            self.step_fn.status.zero_()
            raise StepError(f"a kernel reported inconsistent cache metadata (code {host[-1]})")
        host.pop()
        for req, tok in zip(reqs, host):
            req.output_ids.append(tok)
            if req.state is RequestState.PREFILL:
                req.transition(RequestState.DECODE)
            if req.should_stop():
                req.transition(RequestState.FINISHED)
                self._retire(req)
        return plan

    def generate(self, prompts: Sequence[Sequence[int]], params: SamplingParams | Sequence[SamplingParams]) -> list[list[int]]:
        """Submit all prompts (token ids) at once and run to completion; output token ids per prompt."""
        if isinstance(params, SamplingParams):
            params = [params] * len(prompts)
        reqs = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        while self.has_unfinished:
            if self.step() is None:
                raise RuntimeError("the scheduler produced no step although requests are unfinished")
        return [r.output_ids for r in reqs]
