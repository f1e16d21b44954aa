"""Reads a model folder's safetensors by tensor name into what a model declared.

Follows miniserve/model/weights.py:94-137: every ``*.safetensors`` file of the folder, in sorted
order; tensors go straight to the device; a tied checkpoint may still ship a duplicate head,
which is dropped; anything that does not match the declaration ends in ONE ``ValueError`` that
lists missing and unexpected tensors and wrong shapes. Floating tensors are kept in the run's
dtype (bfloat16 for serving), integer tables as int32; a declaration may ask for float32 or for
"as stored" (a tensor stored in 32-bit stays so).

Two things are data here rather than code. ``rules`` (``config.spec.TensorRule``) say where a
checkpoint's tensor goes when it does not simply carry a declared name: renamed, or cut into
several declared tensors. ``stacks`` say which declared tensors a part wants joined along their
first axis; the joined tensor is allocated once and every piece is read straight into its rows, so
the pieces and the whole are never both alive (at the largest sizes that is several GB per layer
kind).
"""

from __future__ import annotations

from pathlib import Path
from typing import Iterable, Mapping, Sequence

import torch

from ..config.spec import TensorRule
from ..parts.base import WeightDecl

_LIST_LIMIT = 12


class CheckpointMismatch(ValueError):
    """The checkpoint does not match the model's declaration. ``missing``, ``unexpected`` and
    ``wrong_shape`` hold the complete lists; the message shows the first few of each."""

    def __init__(self, path, missing, unexpected, wrong_shape):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong_shape

        def show(items):
            items = list(items)
            more = f" ... and {len(items) - _LIST_LIMIT} more" if len(items) > _LIST_LIMIT else ""
            return f"[{', '.join(map(str, items[:_LIST_LIMIT]))}{more}]"

        super().__init__(
            f"checkpoint {path} does not match its config: "
            f"{len(missing)} missing {show(missing)}; {len(unexpected)} unexpected {show(unexpected)}; "
            f"{len(wrong_shape)} with a wrong shape {show(wrong_shape)}")


def _target_dtype(decl: WeightDecl, stored: torch.dtype, run_dtype: torch.dtype) -> torch.dtype:
    if decl.precision == "int32":
        return torch.int32
    if decl.precision == "float32":
        return torch.float32
    if decl.precision == "stored" and stored in (torch.float32, torch.int32):
        return stored
    return run_dtype


class StackPlan:
    """Where the pieces of joined tensors go: ``place[piece] = (joined name, first row)``."""

    def __init__(self, decls: Mapping[str, WeightDecl], stacks: Mapping[str, Sequence[str]] | None):
        self.place: dict[str, tuple[str, int]] = {}
        self.shape: dict[str, tuple[int, ...]] = {}
        self.pieces: dict[str, tuple[str, ...]] = {}
        for joined, pieces in (stacks or {}).items():
            if any(p not in decls for p in pieces):
                continue  # a stack of tensors nobody declared: nothing to join
            tail = {tuple(decls[p].shape[1:]) for p in pieces}
            kinds = {decls[p].precision for p in pieces}
            if len(tail) != 1 or len(kinds) != 1:
                raise ValueError(f"the pieces of {joined} differ in shape or precision: {list(pieces)}")
            row = 0
            for p in pieces:
                self.place[p] = (joined, row)
                row += decls[p].shape[0]
            self.shape[joined] = (row, *tail.pop())
            self.pieces[joined] = tuple(pieces)


def load_weights(model_dir: str | Path, decls: Mapping[str, WeightDecl], dtype: torch.dtype,
                 device: torch.device | str, ignorable: Iterable[str] = (), rules: Sequence[TensorRule] = (),
                 stacks: Mapping[str, Sequence[str]] | None = None) -> dict[str, torch.Tensor]:
    """``decls``: full tensor name -> declaration. ``ignorable``: names that may be present
    without being declared (the duplicate head of a tied checkpoint). Returns the declared
    tensors by name, except that the pieces of a stack come back joined under the stack's name."""
    from safetensors import safe_open

    model_dir = Path(model_dir)
    files = sorted(model_dir.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors files in {model_dir}")
    ignorable = set(ignorable)
    by_source = {r.source: r for r in rules}
    plan = StackPlan(decls, stacks)
    found: dict[str, torch.Tensor] = {}
    seen: set[str] = set()
    unexpected: list[str] = []
    wrong: list[str] = []

    def deliver(name: str, t: torch.Tensor, origin: str) -> None:
        """One declared tensor's values have arrived (``t`` may be a view of a larger tensor)."""
        decl = decls[name]
        if tuple(t.shape) != tuple(decl.shape):
            wrong.append(f"{origin}: {tuple(t.shape)} != {tuple(decl.shape)}")
            seen.add(name)
            return
        want = _target_dtype(decl, t.dtype, dtype)
        seen.add(name)
        if name in plan.place:
            joined, row = plan.place[name]
            if joined not in found:
                found[joined] = torch.empty(plan.shape[joined], dtype=want, device=device)
            found[joined][row:row + t.shape[0]].copy_(t)
        else:
            found[name] = t.to(want).contiguous()

    for f in files:
        with safe_open(str(f), framework="pt", device=str(device)) as sf:
            for source in sf.keys():
                rule = by_source.get(source)
                targets = rule.targets if rule is not None else ((source, -1),)
                if rule is None and source not in decls:
                    if source not in ignorable:
                        unexpected.append(source)
                    continue
                undeclared = [n for n, _ in targets if n not in decls]
                if undeclared:
                    unexpected.append(f"{source} (maps to undeclared {undeclared})")
                    continue
                if len(targets) == 1 and targets[0][1] < 0:
                    # the cheap check first: a tensor of the wrong shape is not read at all
                    shape = tuple(sf.get_slice(source).get_shape())
                    name = targets[0][0]
                    if shape != tuple(decls[name].shape):
                        wrong.append(f"{source}: {shape} != {tuple(decls[name].shape)}")
                        seen.add(name)
                        continue
                    deliver(name, sf.get_tensor(source), source)
                    continue
                rows = sum(r for _, r in targets)
                shape = tuple(sf.get_slice(source).get_shape())
                if not shape or shape[0] != rows:
                    wrong.append(f"{source}: {shape} cannot be cut into rows {[r for _, r in targets]}")
                    seen.update(n for n, _ in targets)
                    continue
                whole, at = sf.get_tensor(source), 0
                for name, r in targets:
                    deliver(name, whole[at:at + r], f"{source}[{at}:{at + r}] -> {name}")
                    at += r
    missing = sorted(set(decls) - seen)
    if missing or unexpected or wrong:
        raise CheckpointMismatch(model_dir, missing, sorted(unexpected), sorted(wrong))
    return found
