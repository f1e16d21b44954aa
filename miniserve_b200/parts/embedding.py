"""Token embedding and the output head."""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, WeightDecl, param, register_part


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    """h = table[ids] (miniserve/model/qwen3.py:211), widened to the float32 residual stream.
    Parameters: ``vocab``, ``hidden``, ``name`` (the tensor's full name)."""
    shape_static = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab = param(spec, "vocab", int)
        self.hidden = param(spec, "hidden", int)
        self.name = param(spec, "name", str)

    def weights(self):
        return {self.name: WeightDecl((self.vocab, self.hidden))}

    def bind(self, tensors):
        self.table = tensors[self.name].contiguous()

    def forward(self, ctx) -> torch.Tensor:
        residual = torch.empty((ctx.num_tokens, self.hidden), dtype=torch.float32, device=self.table.device)
        ops.embed_gather(residual, self.table, ctx.token_ids, stream=ctx.stream)
        return residual



@register_part("head", "linear_head")
class LinearHead(Part):
    """logits = x @ W^T, no bias (miniserve/model/qwen3.py:186); with ``tied`` the matrix is the
    embedding table itself and no tensor of its own is read (miniserve/model/weights.py:116-119,
    135-136). Logits are returned in float32. Parameters: ``vocab``, ``hidden``, ``tied``,
    ``name``, ``tied_to``."""
    shape_static = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab = param(spec, "vocab", int)
        self.hidden = param(spec, "hidden", int)
        self.tied = bool(spec.get("tied", False))
        self.name = param(spec, "name", str)
        self.tied_to = spec.get("tied_to")
        if self.tied and not self.tied_to:
            raise ValueError("a tied head needs 'tied_to', the name of the embedding tensor")

    def weights(self):
        return {} if self.tied else {self.name: WeightDecl((self.vocab, self.hidden))}

    def bind(self, tensors):
        if not self.tied:
            self.weight = tensors[self.name].contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        logits = torch.empty((x.shape[0], self.vocab), dtype=torch.float32, device=x.device)
        if x.shape[0]:
            ops.linear(x, self.weight, out=logits, stream=ctx.stream)
        return logits
