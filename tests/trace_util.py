"""Helpers for the replay tests: build traces, run bin/trace_run, collect logits by
(request, position), and compute the plain implementation's logits for the same tokens."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

from tests.plain import qwen3_plain as plain

ROOT = Path(__file__).resolve().parent.parent
TRACE_RUN = ROOT / "bin" / "trace_run"


class Trace:
    """A list of steps plus the bookkeeping to map output rows back to (request, position)."""

    def __init__(self):
        self.steps: list[dict] = []
        self.wanted: list[list[tuple[str, int]]] = []  # per step: (request id, absolute position) per output row
        self.progress: dict[str, int] = {}
        self.live: set[str] = set()
        self.max_live_tokens = 0
        self.held: dict[str, int] = {}

    def step(self, entries: list[tuple[str, list[int], list[int] | str]], end: list[str] = ()):
        """entries: (id, tokens, want) with want a list of indices into tokens, or "all" / "last"."""
        ents, wanted = [], []
        for rid, tokens, want in entries:
            start = self.progress.get(rid, 0)
            if want == "all":
                want = list(range(len(tokens)))
            elif want == "last":
                want = [len(tokens) - 1]
            ents.append({"id": rid, "tokens": list(tokens), "want": list(want)})
            wanted += [(rid, start + w) for w in want]
            self.progress[rid] = start + len(tokens)
            self.live.add(rid)
            self.held[rid] = self.progress[rid]
        assert len(self.live) <= 4, "at most four requests are live at a time"
        self.max_live_tokens = max(self.max_live_tokens, sum(-(-n // 64) * 64 for n in self.held.values()))
        self.steps.append({"step": len(self.steps), "entries": ents, "end": list(end)})
        self.wanted.append(wanted)
        for rid in end:
            self.live.discard(rid)
            self.held.pop(rid, None)
            self.progress.pop(rid, None)

    def text(self) -> str:
        return "".join(json.dumps(s) + "\n" for s in self.steps)


def run_trace(model_dir, dtype: str, trace: Trace, out_dir, max_tokens: int | None = None, page_size: int | None = None,
              vocab: int | None = None, env: dict | None = None) -> dict[tuple[str, int, int], torch.Tensor]:
    """Run bin/trace_run on ``trace``; returns {(request id, position, step): logits}."""
    out_dir = Path(out_dir)
    cmd = [sys.executable, str(TRACE_RUN), "--model", str(model_dir), "--dtype", dtype, "--out", str(out_dir),
           "--max-tokens", str(max_tokens if max_tokens is not None else trace.max_live_tokens)]
    if page_size is not None:
        cmd += ["--page-size", str(page_size)]
    proc = subprocess.run(cmd, input=trace.text(), capture_output=True, text=True, env=env or os.environ.copy(),
                          timeout=900)
    assert proc.returncode == 0, f"trace_run failed ({proc.returncode}):\n{proc.stderr[-4000:]}"
    done = [line for line in proc.stdout.splitlines() if line.startswith("done ")]
    assert done == [f"done {s['step']}" for s in trace.steps], proc.stdout[-2000:]
    if vocab is None:
        vocab = json.loads((Path(model_dir) / "config.json").read_text())["vocab_size"]
    result = {}
    for s, wanted in zip(trace.steps, trace.wanted):
        path = out_dir / f"{s['step']}.f32"
        if not wanted:
            assert not path.exists()
            continue
        arr = np.fromfile(path, dtype="<f4").reshape(len(wanted), vocab)
        for (rid, pos), row in zip(wanted, arr):
            result[(rid, pos, s["step"])] = torch.from_numpy(row.copy())
    return result


def plain_logits(model_dir, sequences: dict[str, list[int]]) -> dict[str, torch.Tensor]:
    """float32 logits of the plain implementation at every position of every sequence."""
    cfg, w = plain.read_config(model_dir), plain.read_weights(model_dir, torch.float32)
    return {k: plain.all_logits(cfg, w, ids) for k, ids in sequences.items()}


def bfloat16_noise(model_dir, sequences: dict[str, list[int]], expect: dict[str, torch.Tensor]) -> tuple[float, float]:
    """How far the plain implementation itself moves when it runs in bfloat16 instead of float32
    on these sequences: (largest, mean over positions) of the per-position largest logit
    difference. This is what rounding to bfloat16 costs on this model and these inputs."""
    cfg, w = plain.read_config(model_dir), plain.read_weights(model_dir, torch.bfloat16)
    errs = torch.cat([(plain.all_logits(cfg, w, ids).float() - expect[k]).abs().max(dim=1).values
                      for k, ids in sequences.items()])
    return errs.max().item(), errs.mean().item()


def check_bfloat16(errors: torch.Tensor, noise: tuple[float, float], what: str = "") -> None:
    """``errors``: per position, the engine's largest logit difference from the float32 truth.
    The engine keeps more in float32 than a plain bfloat16 run does, so on average it must be
    at least as near to the truth; a single position may be up to twice the plain run's worst
    (both are the largest of many random rounding errors). A dropped, stale or misplaced key
    moves logits by the size of the logits themselves, far beyond either bound."""
    worst, mean = noise
    assert errors.mean().item() <= mean, f"{what}: mean error {errors.mean().item():.3e} above bfloat16 noise {mean:.3e}"
    assert errors.max().item() <= 2 * worst, (
        f"{what}: position {int(errors.argmax())} is off by {errors.max().item():.3e}, bfloat16 noise peaks at {worst:.3e}")


def sharpen_attention(model_dir, factor: float = 2.5) -> None:
    """Scale the q/k norm weights of a model folder so that attention is peaked rather than near
    uniform: a key that is dropped, misplaced or stale then moves the logits visibly."""
    from safetensors.torch import load_file, save_file

    path = Path(model_dir) / "model.safetensors"
    tensors = load_file(str(path))
    for k in list(tensors):
        if k.endswith("q_norm.weight") or k.endswith("k_norm.weight"):
            tensors[k] = (tensors[k].float() * factor).to(tensors[k].dtype)
    save_file(tensors, str(path))
