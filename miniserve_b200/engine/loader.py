"""From a model folder (or a preset and a seed) to a model with its weights on the device."""

from __future__ import annotations

from pathlib import Path
from typing import Any, Mapping

import torch

from ..config.registry import load_config_dict, resolve
from ..parts.decoder import DecoderModel
from ..weights.loader import load_weights
from ..weights.random_init import random_tensors

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(dtype: str | torch.dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype}")
        return dtype
    try:
        return DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(DTYPES)}, got {dtype!r}") from None


def _ignorable(model: DecoderModel) -> set[str]:
    head = model.head
    return {head.name} if getattr(head, "tied", False) else set()


def load_model(model_dir: str | Path, dtype: str | torch.dtype = "bfloat16",
               device: str | torch.device = "cuda") -> tuple[dict, Any, DecoderModel]:
    """(raw config.json, typed configuration, model) for a folder with config.json and
    safetensors; the model class is chosen by ``architectures`` in config.json."""
    raw = load_config_dict(model_dir)
    _, cfg, spec = resolve(raw)
    model = DecoderModel(spec, parse_dtype(dtype), device)
    tensors = load_weights(model_dir, model.weight_decls(), model.dtype, model.device, ignorable=_ignorable(model),
                           rules=spec.checkpoint_rules, stacks=model.weight_stacks())
    model.bind(tensors)
    return raw, cfg, model


def random_model(raw_config: Mapping[str, Any], seed: int, dtype: str | torch.dtype = "bfloat16",
                 device: str | torch.device = "cuda", std: float = 0.02,
                 draw_on_device: bool = False) -> tuple[dict, Any, DecoderModel]:
    """A model of this configuration with random weights, without going through a folder."""
    raw = dict(raw_config)
    _, cfg, spec = resolve(raw)
    model = DecoderModel(spec, parse_dtype(dtype), device)
    model.bind(random_tensors(model.weight_decls(), seed, dtype=model.dtype, std=std, device=model.device,
                              draw_on_device=draw_on_device, stacks=model.weight_stacks()))
    return raw, cfg, model
