"""Position encodings that act on q and k inside the attention mixer."""

from __future__ import annotations

import torch

from .base import Part, param, register_part


@register_part("position", "rope_neox")
class RotaryNeox(Part):
    """Rotate-half rotary encoding: inv_freq[j] = 1 / theta^(2j / rotary_dim), computed on the
    CPU in float32 from an int64 arange exactly as the reference does
    (miniserve/model/qwen3.py:98-101); the kernel multiplies by the position and takes
    cos/sin in float32. Parameters: ``head_dim``, ``theta``, optional ``rotary_dim``."""
    shape_static = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.head_dim = param(spec, "head_dim", int)
        self.theta = param(spec, "theta", float)
        self.rotary_dim = int(spec.get("rotary_dim") or self.head_dim)
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim={self.rotary_dim} must be even and at most head_dim={self.head_dim}")
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.int64).to(torch.float32) / self.rotary_dim
        self.inv_freq = (1.0 / (self.theta ** exponent)).to(env.device)

    def kernel_table(self) -> tuple[torch.Tensor | None, int]:
        return self.inv_freq, self.rotary_dim

    def step_table(self, ctx) -> torch.Tensor | None:
        """cos/sin of every token of this step, made once per step and shared by all layers
        whose encoding has the same frequencies (the reference's fused path keeps the same
        float32 table, miniserve/model/fused.py:183-184)."""
        from .. import ops

        key = ("rope_table", self.theta, self.rotary_dim)
        table = ctx.step_cache.get(key)
        if table is None:
            table = ops.rope_table(ctx.positions, self.inv_freq, ctx.num_tokens, self.rotary_dim, stream=ctx.stream)
            ctx.step_cache[key] = table
        return table


@register_part("position", "none")
class NoPosition(Part):
    """No position encoding: q and k pass through unrotated."""
    shape_static = True

    def kernel_table(self):
        return None, 0

    def step_table(self, ctx):
        return None
