"""Requests and their life cycle.

    WAITING -> PREFILL -> DECODE -> FINISHED        any live state -> ABORTED
       ^          |          |
       +------ preempted ----+

The same states and edges as miniserve/engine/request.py:30-60: PREFILL covers every step in
which a portion of the prompt runs; the first output token is sampled by the step that runs the
prompt's last token, so a request can finish straight from PREFILL. A preempted request loses
what it holds in the cache but keeps its output; when it is admitted again it runs
prompt + output as its prompt, and the logits at the last position are those the interrupted
decode step would have produced (miniserve/engine/request.py:15-18).
"""

from __future__ import annotations

import enum
from dataclasses import dataclass, field

from ..cache.manager import RequestCache


class RequestState(enum.Enum):
    WAITING = "waiting"
    PREFILL = "prefill"
    DECODE = "decode"
    FINISHED = "finished"
    ABORTED = "aborted"


_EDGES = {
    # WAITING -> FINISHED: with overlap scheduling, a request preempted before its last sampled
    # token was read back, which then turns out to end it
    RequestState.WAITING: {RequestState.PREFILL, RequestState.ABORTED, RequestState.FINISHED},
    RequestState.PREFILL: {RequestState.DECODE, RequestState.FINISHED, RequestState.ABORTED, RequestState.WAITING},
    RequestState.DECODE: {RequestState.FINISHED, RequestState.ABORTED, RequestState.WAITING},
    RequestState.FINISHED: set(),
    RequestState.ABORTED: set(),
}


# Output slot of a token that was sampled on the device and has not been read back yet
# (overlap scheduling, miniserve/engine/request.py:47).
PLACEHOLDER = -1


class InvalidTransition(RuntimeError):
    pass


@dataclass(frozen=True)
class SamplingParams:
    """Names and meanings of miniserve/engine/request.py:58-80: ``temperature`` 0 is greedy;
    ``top_p`` keeps the smallest set of most likely tokens whose mass reaches it; the stop token
    is kept in the output; ``seed`` None lets the engine assign one."""

    max_new_tokens: int
    stop_token_ids: frozenset[int] = frozenset()
    temperature: float = 0.0
    top_p: float = 1.0
    seed: int | None = None

    def __post_init__(self):
        object.__setattr__(self, "stop_token_ids", frozenset(self.stop_token_ids))
        if self.max_new_tokens < 1:
            raise ValueError(f"max_new_tokens must be >= 1, got {self.max_new_tokens}")
        if not self.temperature >= 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if not 0 < self.top_p <= 1:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.seed is not None and not 0 <= self.seed < 2 ** 32:
            raise ValueError(f"seed must be in [0, 2**32), got {self.seed}")

    @property
    def is_greedy(self) -> bool:
        return self.temperature == 0


@dataclass(eq=False)
class Request:
    rid: int
    prompt_ids: list[int]
    params: SamplingParams
    output_ids: list[int] = field(default_factory=list)
    state: RequestState = RequestState.WAITING
    cache: RequestCache | None = None  # held between admission and release
    seed: int = 0
    num_preemptions: int = 0
    num_pending: int = 0  # trailing PLACEHOLDER entries of output_ids

    def __post_init__(self):
        if not self.prompt_ids:
            raise ValueError("empty prompt")

    def transition(self, new: RequestState) -> None:
        if new not in _EDGES[self.state]:
            raise InvalidTransition(f"request {self.rid}: {self.state.name} -> {new.name}")
        self.state = new

    @property
    def is_done(self) -> bool:
        return self.state in (RequestState.FINISHED, RequestState.ABORTED)

    @property
    def seq_len(self) -> int:
        """Tokens a prefill of this request runs: the prompt and any output kept across a preemption."""
        return len(self.prompt_ids) + len(self.output_ids)

    @property
    def max_len(self) -> int:
        return len(self.prompt_ids) + self.params.max_new_tokens

    @property
    def num_cached(self) -> int:
        return self.cache.num_tokens if self.cache is not None else 0

    @property
    def reached_max_tokens(self) -> bool:
        return len(self.output_ids) >= self.params.max_new_tokens

    def token_slice(self, start: int, n: int) -> list[int]:
        """Tokens start .. start+n of prompt + output."""
        p = len(self.prompt_ids)
        if start >= p:
            return self.output_ids[start - p:start - p + n]
        if start + n <= p:
            return self.prompt_ids[start:start + n]
        return self.prompt_ids[start:] + self.output_ids[:start + n - p]

    @property
    def ready_ids(self) -> list[int]:
        """Output tokens read back so far."""
        return self.output_ids[:len(self.output_ids) - self.num_pending]

    def drop_pending(self) -> None:
        """Forget tokens sampled after the request ended (launched before its end was known)."""
        if self.num_pending:
            del self.output_ids[-self.num_pending:]
            self.num_pending = 0

    def should_stop(self) -> bool:
        return self.reached_max_tokens or (bool(self.output_ids) and self.output_ids[-1] in self.params.stop_token_ids)
