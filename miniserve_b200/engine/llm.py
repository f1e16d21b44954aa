"""The Python entry point: a model folder (or a preset with random weights) in, token ids out.

The reference's entry point is ``Engine(model, **kwargs).generate(prompts, params)`` on token
ids, with no tokenizer on that path (miniserve/engine/engine.py:206-211); ``LLM`` adds the
loading in front of it.
"""

from __future__ import annotations

from pathlib import Path
from typing import Sequence

import torch

from ..config.presets import preset
from .engine import Engine
from .loader import load_model, random_model
from .request import SamplingParams


class LLM:
    def __init__(self, model: str | Path | None = None, *, random: str | dict | None = None, weights_seed: int = 0,
                 dtype: str | torch.dtype = "bfloat16", device: str = "cuda:0", **engine_kwargs):
        """``model``: a folder with config.json and safetensors. ``random``: instead of a folder,
        a preset name (``tiny-a``, ``tiny-b``, ``0.6b``, ``1.7b``, ``8b``, ``32b``) or a
        config.json dict, filled with random weights from ``weights_seed``. The remaining
        keywords are the engine's (``kv_pool_tokens``, ``page_size``, ``max_running``,
        ``max_prefill_tokens``, ``chunked_prefill_size``, ``seed``, ``cuda_graph``,
        ``cuda_graph_max_bs``, ``step_graphs``, ``overlap``)."""
        if (model is None) == (random is None):
            raise ValueError("give either a model folder or random=PRESET")
        if model is not None:
            self.raw_config, self.config, self.model = load_model(model, dtype, device)
        else:
            raw = preset(random) if isinstance(random, str) else dict(random)
            big = raw.get("hidden_size", 0) * raw.get("num_hidden_layers", 0) > 4096
            self.raw_config, self.config, self.model = random_model(raw, weights_seed, dtype, device,
                                                                    draw_on_device=big)
        self.engine = Engine(self.model, **engine_kwargs)

    def generate(self, prompts: Sequence[Sequence[int]], params: SamplingParams | Sequence[SamplingParams]) -> list[list[int]]:
        return self.engine.generate(prompts, params)
