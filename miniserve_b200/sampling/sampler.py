"""Per-step sampling arguments and the call into the sampling kernels.

As in miniserve/engine/sampler.py:65-100: a step whose rows are all greedy takes the plain
argmax; otherwise every row gets (temperature, top_p, seed, counter) with counter = the index
of the token being sampled in its sequence, so that a request draws the same noise wherever it
sits in a batch and whether or not it was preempted and run again. Tokens stay on the device;
the engine copies them back once per step.
"""

from __future__ import annotations

from typing import Sequence

import torch

from .. import ops


class Sampler:
    def __init__(self, device: torch.device | str, vocab_size: int, max_rows: int = 64):
        self.device = torch.device(device)
        self.vocab_size = vocab_size
        self._scratch = None
        self._cap = 0
        self._ensure(max_rows)

    def _ensure(self, rows: int) -> None:
        if rows <= self._cap:
            return
        self._cap = max(rows, 2 * self._cap)
        self._scratch = torch.empty(self._cap * ops.nucleus_bytes(), dtype=torch.uint8, device=self.device)

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float] | None = None,
               top_ps: Sequence[float] | None = None, seeds: Sequence[int] | None = None,
               counters: Sequence[int] | None = None, stream=None) -> torch.Tensor:
        """``logits`` float32 [rows, vocab] -> int32 [rows] on the device."""
        rows = logits.shape[0]
        tokens = torch.empty(rows, dtype=torch.int32, device=self.device)
        if rows == 0:
            return tokens
        if temperatures is None or all(t == 0 for t in temperatures):
            ops.sample(tokens, logits, stream=stream)
            return tokens
        self._ensure(rows)
        f32 = torch.tensor([list(temperatures), list(top_ps or [1.0] * rows)], dtype=torch.float32).pin_memory()
        i64 = torch.tensor([list(seeds), list(counters)], dtype=torch.int64).pin_memory()
        f32 = f32.to(self.device, non_blocking=True)
        i64 = i64.to(self.device, non_blocking=True)
        use_top_p = top_ps is not None and any(p < 1 for p in top_ps)
        ops.sample(tokens, logits, temperature=f32[0], top_p=f32[1] if use_top_p else None, seed=i64[0],
                   counter=i64[1], scratch=self._scratch if use_top_p else None, stream=stream)
        return tokens
