"""Random weights from a configuration and a seed.

The reference has no such mode; its nearest thing is ``torch.randn(shape)`` per expected
tensor in a test (tests/test_weights.py:27). Here matrices are N(0, std) and norm scales
1 + N(0, 0.1). Values are drawn on the CPU in float32 in declaration order, so a seed gives
the same model everywhere; ``write_model_folder`` stores them as a normal model folder
(config.json + model.safetensors) that the ordinary loader reads back.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping, Sequence

import torch

from ..parts.base import WeightDecl


def random_tensors(decls: Mapping[str, WeightDecl], seed: int, dtype: torch.dtype = torch.bfloat16,
                   std: float = 0.02, device: torch.device | str = "cpu", draw_on_device: bool = False,
                   stacks: Mapping[str, Sequence[str]] | None = None) -> dict[str, torch.Tensor]:
    """``draw_on_device``: draw with the device's generator instead (fast for large models,
    but the values then depend on the device type). ``stacks``: declared tensors that a part
    wants joined (``Part.stacks``); each piece is drawn as it would be alone and written straight
    into the joined tensor, which comes back under the stack's name instead of its pieces."""
    from .loader import StackPlan

    gen_device = torch.device(device) if draw_on_device else torch.device("cpu")
    gen = torch.Generator(device=gen_device).manual_seed(seed)
    plan = StackPlan(decls, stacks)
    out: dict[str, torch.Tensor] = {}
    for name, decl in decls.items():
        if decl.precision == "int32":
            t, want = torch.zeros(decl.shape, dtype=torch.int32, device=device), torch.int32
        else:
            t = torch.randn(decl.shape, generator=gen, dtype=torch.float32, device=gen_device)
            t = (1.0 + 0.1 * t) if decl.init == "ones_normal" else std * t
            want = torch.float32 if decl.precision in ("float32", "stored") else dtype
        if name in plan.place:
            joined, row = plan.place[name]
            if joined not in out:
                out[joined] = torch.empty(plan.shape[joined], dtype=want, device=device)
            out[joined][row:row + decl.shape[0]].copy_(t)
        else:
            out[name] = t.to(device=device, dtype=want).contiguous()
    return out


def write_model_folder(folder: str | Path, raw_config: Mapping[str, Any], seed: int,
                       dtype: torch.dtype = torch.bfloat16, std: float = 0.02) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for a random model of this configuration."""
    from safetensors.torch import save_file

    from ..config.registry import resolve
    from ..parts.decoder import DecoderModel

    _, _, spec = resolve(raw_config)
    decls = DecoderModel(spec, dtype, "cpu").weight_decls()
    tensors = random_tensors(decls, seed, dtype=dtype, std=std)
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(dict(raw_config), indent=1))
    save_file(tensors, str(folder / "model.safetensors"))
    return folder
