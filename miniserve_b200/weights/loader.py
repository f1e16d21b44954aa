"""Reads a model folder's safetensors by tensor name into what a model declared.

Follows miniserve/model/weights.py:94-137: every ``*.safetensors`` file of the folder, in sorted
order; tensors go straight to the device; a tied checkpoint may still ship a duplicate head,
which is dropped; anything that does not match the declaration ends in ONE ``ValueError`` that
lists missing and unexpected tensors and wrong shapes. Floating tensors are kept in the run's
dtype (bfloat16 for serving), integer tables as int32; a declaration may ask for float32 or for
"as stored" (a tensor stored in 32-bit stays so).
"""

from __future__ import annotations

from pathlib import Path
from typing import Iterable, Mapping

import torch

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


def load_weights(model_dir: str | Path, decls: Mapping[str, WeightDecl], dtype: torch.dtype,
                 device: torch.device | str, ignorable: Iterable[str] = ()) -> dict[str, torch.Tensor]:
    """``decls``: full tensor name -> declaration. ``ignorable``: names that may be present
    without being declared (the duplicate head of a tied checkpoint)."""
    from safetensors import safe_open

    model_dir = Path(model_dir)
    files = sorted(model_dir.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors files in {model_dir}")
    ignorable = set(ignorable)
    found: dict[str, torch.Tensor] = {}
    unexpected: list[str] = []
    wrong: list[str] = []
    for f in files:
        with safe_open(str(f), framework="pt", device=str(device)) as sf:
            for name in sf.keys():
                decl = decls.get(name)
                if decl is None:
                    if name not in ignorable:
                        unexpected.append(name)
                    continue
                shape = tuple(sf.get_slice(name).get_shape())
                if shape != tuple(decl.shape):
                    wrong.append(f"{name}: {shape} != {tuple(decl.shape)}")
                    continue
                t = sf.get_tensor(name)
                found[name] = t.to(_target_dtype(decl, t.dtype, dtype)).contiguous()
    missing = sorted(set(decls) - set(found) - {w.split(":")[0] for w in wrong})
    if missing or unexpected or wrong:
        raise CheckpointMismatch(model_dir, missing, sorted(unexpected), sorted(wrong))
    return found
