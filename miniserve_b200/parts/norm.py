"""RMSNorm with the residual add (and an optional row gather) fused in."""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, WeightDecl, param, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    """y = x * rsqrt(mean(x^2) + eps) * weight, statistics in float32, no bias and no ``1 +``
    offset (miniserve/model/qwen3.py:78-82). Parameters: ``size``, ``eps``."""
    shape_static = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = param(spec, "size", int)
        self.eps = param(spec, "eps", float)

    def weights(self):
        return {"weight": WeightDecl((self.size,), init="ones_normal")}

    def forward(self, residual: torch.Tensor, delta: torch.Tensor | None, ctx, rows: torch.Tensor | None = None,
                num_rows: int | None = None, write_residual: bool = True) -> torch.Tensor:
        """Normalise ``residual (+ delta)``; without ``rows`` the sum is stored back into
        ``residual``. With ``rows`` (int32 indices) only those rows are produced."""
        n = residual.shape[0] if rows is None else (num_rows if num_rows is not None else rows.numel())
        out = ctx.buffer("norm.out", (n, self.size), self.env.dtype, residual.device)
        ops.add_rmsnorm(out, residual, delta, self.w_weight, self.eps, rows=rows, num_rows=n,
                        write_residual=write_residual, stream=ctx.stream)
        return out
