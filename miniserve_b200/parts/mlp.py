"""Dense gated feed-forward."""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, WeightDecl, param, register_part


@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    """down(silu(gate(x)) * up(x)), no biases (miniserve/model/qwen3.py:128-131). The gate and
    up matrices are stacked at load so that one product makes both
    (miniserve/model/fused.py:41-95 does the same). Parameters: ``hidden``, ``intermediate``."""
    shape_static = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = param(spec, "hidden", int)
        self.inter = param(spec, "intermediate", int)

    def weights(self):
        return {
            "gate_proj.weight": WeightDecl((self.inter, self.hidden)),
            "up_proj.weight": WeightDecl((self.inter, self.hidden)),
            "down_proj.weight": WeightDecl((self.hidden, self.inter)),
        }

    def stacks(self):
        return {"gate_up_proj.weight": ("gate_proj.weight", "up_proj.weight")}

    def bind(self, tensors):
        self.w_gate_up = self.joined(tensors, "gate_up_proj.weight", self.stacks()["gate_up_proj.weight"])
        self.w_down = tensors["down_proj.weight"].contiguous()

    def forward(self, x, ctx) -> torch.Tensor:
        t, dt, dev = x.shape[0], self.env.dtype, self.w_down.device
        act = ctx.buffer("mlp.act", (t, self.inter), dt, dev)
        if dt == torch.bfloat16:
            # one kernel with the activation in its epilogue where there is one (decode steps, wide prompt steps)
            fused = ops.silu_mul_is_fused(x, self.w_gate_up, act)
            scratch = None if fused else ctx.buffer("mlp.gate_up", (t, 2 * self.inter), dt, dev)
            ops.linear_silu_mul(x, self.w_gate_up, act, scratch=scratch, stream=ctx.stream)
        else:
            gate_up = ops.linear(x, self.w_gate_up, stream=ctx.stream, out=ctx.buffer("mlp.gate_up", (t, 2 * self.inter), dt, dev))
            ops.silu_mul(act, gate_up, stream=ctx.stream)
        return ops.linear(act, self.w_down, stream=ctx.stream, out=ctx.buffer("mlp.down", (t, self.hidden), dt, dev))
