"""The scheduler: which requests run in the next step, and with how many tokens each.

Decisions, following miniserve/engine/scheduler.py:

* With a chunk budget (``chunked_prefill_size`` tokens per step, the default): decode first.
  Every decoding request gets its one token; what is left of the budget goes to portions of
  prompts, first of requests already part-way through theirs (in admission order), then of newly
  admitted ones in arrival order (:227-279).
* Without (``chunked_prefill_size=0``): prefill first. Waiting requests are admitted whole under
  ``max_prefill_tokens`` (the first always); a step holds either whole prompts or decode tokens
  (:156-201).
* Admission needs the pages of the whole prompt plus one token, on top of what every running
  request may still allocate; it stops at the first request that does not fit: no skipping ahead
  (:249-257, 294-303). A request that could never fit in the pool is rejected when it is added
  (:143-154).
* When pages run out: requests are preempted, newest admitted first and never the oldest running
  one, until what the rest may still allocate fits. A preempted request gives back everything it
  holds, keeps its output, and goes to the front of the waiting queue to be run again from its
  first token (:281-323). So the oldest request always progresses and nothing deadlocks.

* Two policies decide the order in which waiting requests are tried and who is preempted
  (miniserve/engine/policy.py:44-69): ``fcfs``, arrival order and the newest admitted request as
  above; ``sjf``, least remaining work first (the prompt tokens still to compute plus the tokens the
  request may still generate) and the request with the most remaining work preempted. Under both,
  admission stops at the first request in its order that does not fit, and the oldest running
  request is never preempted. The reference's third policy orders by what a prefix cache holds;
  there is none here.

Budgets are per cache group (a tuple of page counts) and include the slot for per-request state.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from ..cache.manager import CacheManager
from .request import Request, RequestState


def remaining_work(r: Request) -> int:
    """Prompt (and, after a preemption, output) tokens still to compute, plus the tokens the request may
    still generate: what the shortest-job-first policy orders by (miniserve/engine/policy.py:53-56)."""
    return r.seq_len - r.num_cached + r.params.max_new_tokens - len(r.output_ids)


POLICIES = ("fcfs", "sjf")


@dataclass
class PlanRow:
    request: Request
    start: int  # tokens of the request already in the cache
    count: int  # new tokens this step

    @property
    def completes(self) -> bool:
        """The row reaches the end of its sequence, so a token is sampled from its last position."""
        return self.start + self.count == self.request.seq_len


@dataclass
class Plan:
    rows: list[PlanRow]
    num_decode: int  # rows[:num_decode] are single decode tokens
    preempted: list[Request] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(r.count for r in self.rows)

    @property
    def phase(self) -> str:
        if self.num_decode == len(self.rows):
            return "decode"
        return "prefill" if self.num_decode == 0 else "mixed"


def _add(a: tuple[int, ...], b: tuple[int, ...]) -> tuple[int, ...]:
    return tuple(x + y for x, y in zip(a, b))


class Scheduler:
    def __init__(self, cache: CacheManager, max_running: int = 64, max_prefill_tokens: int = 8192,
                 chunked_prefill_size: int = 2048, policy: str = "fcfs"):
        if policy not in POLICIES:
            raise ValueError(f"unknown schedule policy {policy!r}; choose from {list(POLICIES)}")
        self.policy = policy
        if max_running < 1 or max_prefill_tokens < 1:
            raise ValueError("max_running and max_prefill_tokens must be positive")
        if chunked_prefill_size < 0:
            raise ValueError(f"chunked_prefill_size must be >= 0, got {chunked_prefill_size}")
        if max_running > cache.max_requests:
            raise ValueError(f"max_running={max_running} exceeds the cache's {cache.max_requests} request slots")
        self.cache = cache
        self.max_running = max_running
        self.max_prefill_tokens = max_prefill_tokens
        self.chunked_prefill_size = chunked_prefill_size
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []  # admission order
        self.num_preemptions = 0
        self.num_preempted_requests = 0  # requests preempted at least once
        self.stats = dict(first_tokens=0, re_tokens=0)

    # ------------------------------------------------------------------ queues
    def add(self, req: Request) -> None:
        if req.state is not RequestState.WAITING:
            raise ValueError(f"request {req.rid} is {req.state.name}, expected WAITING")
        need = self.cache.pages_for(req.max_len)
        if any(n > have for n, have in zip(need, self.cache.group_pages())):
            raise ValueError(f"request {req.rid} needs up to {req.max_len} tokens of cache, "
                             f"the pool holds {self.cache.num_pages * self.cache.page_size}")
        self.waiting.append(req)

    def retire(self, req: Request) -> None:
        if not req.is_done:
            raise ValueError(f"request {req.rid} is {req.state.name}, not done")
        if req in self.running:
            self.running.remove(req)
        elif req in self.waiting:
            self.waiting.remove(req)

    @property
    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ budget arithmetic
    @staticmethod
    def _decodes(r: Request) -> bool:
        return r.state is RequestState.DECODE and not r.reached_max_tokens

    def _zero(self) -> tuple[int, ...]:
        return (0,) * self.cache.num_groups

    def _outstanding(self, reqs) -> tuple[int, ...]:
        """Pages per group that ``reqs`` may still allocate before any of them finishes: one
        token for each decoding request; the rest of the prompt plus one token for each
        request still in its prefill."""
        need = self._zero()
        for r in reqs:
            if self._decodes(r):
                need = _add(need, self.cache.pages_needed(r.cache, 1))
            elif r.state is RequestState.PREFILL:
                need = _add(need, self.cache.pages_outstanding(r.cache, r.seq_len + 1))
        return need

    def _admission_need(self, req: Request) -> tuple[int, ...]:
        return self.cache.pages_for(req.seq_len + 1)

    # ------------------------------------------------------------------ policy
    def _in_order(self) -> list[Request]:
        """The waiting requests in the order admission tries them."""
        if self.policy == "sjf":
            return sorted(self.waiting, key=remaining_work)  # stable: equals keep their arrival order
        return list(self.waiting)

    def _victim(self, candidates: list[Request]) -> Request:
        """Whom to preempt among ``candidates`` (running requests in admission order, the oldest left out)."""
        if self.policy == "sjf":
            return max(reversed(candidates), key=remaining_work)  # among equals the newest admitted
        return candidates[-1]

    # ------------------------------------------------------------------ preemption
    def _preempt(self, req: Request) -> None:
        req.transition(RequestState.WAITING)
        self.cache.release(req.cache)
        req.cache = None
        self.running.remove(req)
        self.waiting.appendleft(req)  # victims are taken newest first, so arrival order is kept
        self.num_preempted_requests += req.num_preemptions == 0
        req.num_preemptions += 1
        self.num_preemptions += 1

    def _make_room(self, pool: list[Request]) -> list[Request]:
        """Preempt until what ``pool`` may still allocate fits into the free pages."""
        preempted: list[Request] = []
        while not self.cache.fits(self._outstanding(pool)):
            # requests that have sampled their last token and only wait for it to be read back cost
            # nothing to preempt (they will never run again): take those first
            spent = [r for r in self.running if r.state is RequestState.DECODE and r.reached_max_tokens]
            if spent:
                victim = spent[-1]
            else:
                candidates = [r for r in pool if r is not self.running[0]]
                if not candidates:
                    raise RuntimeError("a lone request does not fit in the pool")  # add() rejects those
                victim = self._victim(candidates)
            if pool is not self.running and victim in pool:
                pool.remove(victim)
            self._preempt(victim)
            preempted.append(victim)
        return preempted

    # ------------------------------------------------------------------ step assembly
    def schedule(self) -> Plan | None:
        """The next step, or None if nothing can run. Moves admitted requests to PREFILL and
        preempted ones back to WAITING."""
        if self.chunked_prefill_size:
            return self._schedule_chunked()
        return self._schedule_whole()

    def _admit(self, req: Request) -> None:
        req.cache = self.cache.new_request()
        self.waiting.remove(req)
        req.transition(RequestState.PREFILL)
        self.running.append(req)
        self.stats["first_tokens" if req.num_preemptions == 0 else "re_tokens"] += req.seq_len

    def _schedule_chunked(self) -> Plan | None:
        preempted = self._make_room(self.running)
        budget = self.chunked_prefill_size
        rows = [PlanRow(r, r.seq_len - 1, 1) for r in self.running if self._decodes(r)]
        num_decode = len(rows)
        budget -= num_decode
        for r in self.running:
            if r.state is RequestState.PREFILL and budget > 0:
                start = r.num_cached
                n = min(r.seq_len - start, budget)
                rows.append(PlanRow(r, start, n))
                budget -= n
        margin = None  # what the running requests may still allocate: counted once, then kept up to date
        for req in self._in_order():
            if budget <= 0 or len(self.running) >= self.max_running or self.cache.num_free_slots == 0:
                break
            if req.num_pending:  # its last token is not read back yet; its prefill needs it
                break
            if margin is None:
                margin = self._outstanding(self.running)
            if not self.cache.fits(self._admission_need(req), margin=margin):
                break
            self._admit(req)
            margin = _add(margin, self._outstanding((req,)))
            n = min(req.seq_len, budget)
            rows.append(PlanRow(req, 0, n))
            budget -= n
        if not rows:
            return None
        return Plan(rows, num_decode, preempted)

    def _schedule_whole(self) -> Plan | None:
        admitted: list[Request] = []
        budget = self.max_prefill_tokens
        margin = None
        for req in self._in_order():
            if len(self.running) >= self.max_running or self.cache.num_free_slots == 0:
                break
            if req.num_pending:
                break
            if admitted and req.seq_len > budget:  # the first is admitted even over the budget
                break
            if margin is None:
                margin = self._outstanding(self.running)
            if not self.cache.fits(self._admission_need(req), margin=margin):
                break
            self._admit(req)
            margin = _add(margin, self._outstanding((req,)))
            admitted.append(req)
            budget -= req.seq_len
        if admitted:
            return Plan([PlanRow(r, 0, r.seq_len) for r in admitted], 0)
        decoding = [r for r in self.running if self._decodes(r)]
        preempted = self._make_room(decoding)
        if not decoding:
            return None
        return Plan([PlanRow(r, r.seq_len - 1, 1) for r in decoding], len(decoding), preempted)
