"""What a caller asks for (``SamplingParams``) and the engine's record of one request (``Request``).

A request is in exactly one of five states. The scheduler admits a waiting request (it then
prefills, over one or more steps), the step that runs the last token of its sequence samples the
first output token and turns it to decoding, and it ends when it has produced the tokens it was
allowed or a stop token. Running short of pages sends a prefilling or decoding request back to
waiting: it gives up its pages, keeps the output it has, and later prefills prompt + output in
one sequence. Anything not yet ended can be aborted.

              admit            last prompt token           limit or stop token
    WAITING --------> PREFILL -------------------> DECODE ----------------------> FINISHED
       ^                 |                           |
       +------------- out of pages (preempted) ------+           (any of the three) -> ABORTED

Names and meanings of the public fields follow miniserve/engine/request.py:30-155, so that code
written against that engine reads the same here.
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


def _moves(table: str) -> dict[RequestState, frozenset[RequestState]]:
    out = {}
    for line in table.strip().splitlines():
        src, dst = line.split(":")
        out[RequestState[src.strip()]] = frozenset(RequestState[name] for name in dst.split())
    return out


# Where each state may go. PREFILL -> FINISHED: a request allowed a single token ends in the step
# that samples it. WAITING -> FINISHED only happens when steps overlap: a request was preempted
# while its newest token was still on the device, and that token, once read, is its last.
_MOVES = _moves("""
    WAITING:  PREFILL FINISHED ABORTED
    PREFILL:  DECODE FINISHED WAITING ABORTED
    DECODE:   FINISHED WAITING ABORTED
    FINISHED:
    ABORTED:
""")

# Stands in ``output_ids`` for a token that a launched step has sampled but the host has not read yet.
PLACEHOLDER = -1


class InvalidTransition(RuntimeError):
    """A request was asked to move to a state its current state does not lead to."""


@dataclass(frozen=True)
class SamplingParams:
    """How a request's tokens are chosen and when it stops.

    ``max_new_tokens``: the most tokens to produce (at least one). ``stop_token_ids``: producing
    any of these ends the request; the token stays in the output. ``temperature``: 0 picks the most
    likely token, larger values sample from the softened distribution. ``top_p``: sample only among
    the most likely tokens whose probabilities add up to this much. ``seed``: makes sampling
    repeatable; left None, the engine draws one per request from its own seed.
    """

    max_new_tokens: int
    stop_token_ids: frozenset[int] = frozenset()
    temperature: float = 0.0
    top_p: float = 1.0
    seed: int | None = None

    def __post_init__(self):
        object.__setattr__(self, "stop_token_ids", frozenset(self.stop_token_ids))
        problems = [
            (self.max_new_tokens >= 1, f"max_new_tokens={self.max_new_tokens}: a request produces at least one token"),
            (self.temperature >= 0, f"temperature={self.temperature}: cannot be negative (0 is greedy)"),  # NaN fails too
            (0 < self.top_p <= 1, f"top_p={self.top_p}: a probability mass in (0, 1]"),
            (self.seed is None or 0 <= self.seed < 1 << 32, f"seed={self.seed}: an unsigned 32-bit number, or None"),
        ]
        for ok, message in problems:
            if not ok:
                raise ValueError(message)

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
    cache: RequestCache | None = None  # its pages and state slot, from admission until it ends or is preempted
    seed: int = 0
    num_preemptions: int = 0
    num_pending: int = 0  # how many entries at the end of output_ids are still PLACEHOLDER

    def __post_init__(self):
        if len(self.prompt_ids) == 0:
            raise ValueError(f"request {self.rid} has no prompt tokens")

    # ------------------------------------------------------------------ state
    def transition(self, to: RequestState) -> None:
        if to not in _MOVES[self.state]:
            raise InvalidTransition(f"request {self.rid} is {self.state.name} and cannot become {to.name}")
        self.state = to

    @property
    def is_done(self) -> bool:
        return not _MOVES[self.state]  # the two states that lead nowhere

    # ------------------------------------------------------------------ lengths
    @property
    def seq_len(self) -> int:
        """Length of the sequence a (re)admitted request runs: its prompt plus the output it holds."""
        return len(self.prompt_ids) + len(self.output_ids)

    @property
    def max_len(self) -> int:
        """The longest the sequence can get."""
        return len(self.prompt_ids) + self.params.max_new_tokens

    @property
    def num_cached(self) -> int:
        """Tokens of the sequence whose keys and values are in the cache."""
        return 0 if self.cache is None else self.cache.num_tokens

    @property
    def reached_max_tokens(self) -> bool:
        return len(self.output_ids) >= self.params.max_new_tokens

    # ------------------------------------------------------------------ tokens
    def token_slice(self, start: int, n: int) -> list[int]:
        """Tokens ``start .. start + n - 1`` of the sequence prompt + output."""
        split = len(self.prompt_ids)
        end = start + n
        # each list contributes the part of [start, end) that falls into it (possibly nothing)
        return self.prompt_ids[start:end] + self.output_ids[max(start - split, 0):max(end - split, 0)]

    @property
    def ready_ids(self) -> list[int]:
        """The output tokens the host has read (everything before the placeholders)."""
        return self.output_ids[:len(self.output_ids) - self.num_pending]

    def drop_pending(self) -> None:
        """Discard the placeholders: tokens of steps launched before the request was known to have ended."""
        if self.num_pending:
            self.output_ids = self.output_ids[:len(self.output_ids) - self.num_pending]
            self.num_pending = 0

    def should_stop(self) -> bool:
        last = self.output_ids[-1] if self.output_ids else None
        return self.reached_max_tokens or last in self.params.stop_token_ids
