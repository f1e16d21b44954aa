"""Decode steps of a few requests as chains of products in persistent kernels.

A decode step of a small model is a chain of short dependent kernels: each product is one trip
to HBM long, and between two products sit a launch, a norm or an activation. Here the decoder
asks its parts what they would launch and strings the products together
(``ops/decode_chain.py``): from a layer's output projection to the next layer's input projection
is ONE kernel (o -> +residual, norm -> gate|up, SiLU * up -> down -> +residual, norm -> q|k|v), the
mixer's own work (attention over the cache) runs between two chains, and the last chain ends in
the head's product.

No part is named here. A part takes part in chains by offering, beside ``forward``:

``norm``          ``chain_norm() -> (weight [size] bf16, eps) | None``
``mixer``         ``chain_mixer(ctx, cache) -> ChainMixer | None``
``feed_forward``  ``chain_feed_forward() -> ChainFeedForward | None``
``block``         ``chain_layer(ctx, cache) -> ChainLayer | None``
``embedding``     ``chain_table() -> table [vocab, hidden] bf16 | None``
``head``          ``chain_weight() -> weight [vocab, hidden] bf16 | None``

A model in which every part offers these runs its small decode steps this way; any other model,
step or dtype takes the parts' ``forward`` as before. Both compute the same function; they differ
in where bfloat16 roundings fall (see ``csrc/decode_chain.cu``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch

from .. import ops
from ..ops import decode_chain as chain


@dataclass
class ChainMixer:
    """A mixer as two products around work of its own: ``in_weight`` [width_in, hidden] makes the
    mixer's projection of the normed input; ``run(projection [M, width_in], out [M, width_out])``
    launches what the mixer does with it (for attention: per-head norm, rotation, cache write and
    the attention itself); ``out_weight`` [hidden, width_out] makes the addend to the residual."""

    in_weight: torch.Tensor
    out_weight: torch.Tensor
    run: Callable[[torch.Tensor, torch.Tensor], None]


@dataclass
class ChainFeedForward:
    """A gated feed-forward as two products: ``in_weight`` [2 * inter, hidden] (gate rows, then up
    rows) followed by silu(gate) * up, and ``out_weight`` [hidden, inter]."""

    in_weight: torch.Tensor
    out_weight: torch.Tensor


@dataclass
class ChainLayer:
    norm1: tuple[torch.Tensor, float]
    mixer: ChainMixer
    norm2: tuple[torch.Tensor, float]
    feed_forward: ChainFeedForward


class DecodeChain:
    """Runs a decode step of ``model`` (``parts/decoder.py``) as chains, if the step and every
    part allow it."""

    def __init__(self, model):
        self.model = model
        self.sync_state: torch.Tensor | None = None
        self.launches = 0

    def takes(self, ctx) -> bool:
        m = self.model
        if not ops.DECODE_CHAIN or m.dtype != torch.bfloat16 or not ctx.decode_only:
            return False
        if ctx.num_rows != ctx.num_tokens or not 1 <= ctx.num_tokens <= chain.MAX_ROWS:
            return False
        return all(hasattr(layer, "chain_layer") for layer in m.layers) and hasattr(m.embedding, "chain_table") \
            and hasattr(m.final_norm, "chain_norm") and hasattr(m.head, "chain_weight")

    def run(self, ctx, caches) -> torch.Tensor | None:
        """Logits [wanted, vocab] of the step, or None if some part declined (nothing was launched)."""
        m = self.model
        table, head_w, final = m.embedding.chain_table(), m.head.chain_weight(), m.final_norm.chain_norm()
        if table is None or head_w is None or final is None:
            return None
        layers: list[ChainLayer] = []
        for i, entry in enumerate(m.spec.run_order):
            layer = m.layers[entry.layer].chain_layer(ctx, caches[i])
            if layer is None:
                return None
            layers.append(layer)
        rows, hidden, dev = ctx.num_tokens, m.spec.hidden_size, m.device
        widths = [hidden] + [w.shape[1] for l in layers for w in (l.mixer.out_weight, l.feed_forward.out_weight)]
        if not layers or not chain.fits(rows, max(widths)):
            return None
        if self.sync_state is None:
            self.sync_state = torch.zeros(4, dtype=torch.int32, device=dev)
        ctx.scratch.setdefault("chain_sync", self.sync_state)  # zeroed with the other tickets after a raised status word
        bf16, f32 = torch.bfloat16, torch.float32
        residual = ctx.buffer("chain.residual", (rows, hidden), f32, dev)
        # what a norm needs of the residual: its weighted copy and the sums of squares; one pair for the
        # norms before mixers (written by the embedding and by every down projection), one for those before
        # feed-forwards (written by every output projection)
        xw_a = ctx.buffer("chain.xw_a", (rows, hidden), bf16, dev)
        xw_b = ctx.buffer("chain.xw_b", (rows, hidden), bf16, dev)
        parts = chain.tiles(hidden)
        ss_0 = ctx.buffer("chain.ss_0", (rows, 1), f32, dev)
        ss_a = ctx.buffer("chain.ss_a", (rows, parts), f32, dev)
        ss_b = ctx.buffer("chain.ss_b", (rows, parts), f32, dev)
        chain.embed(residual, xw_a, ss_0, table, ctx.token_ids, layers[0].norm1[0], ctx.stream)
        self.launches = 1
        pending: list[chain.Phase] = []
        ss_in = ss_0
        for i, layer in enumerate(layers):
            mx, ff = layer.mixer, layer.feed_forward
            proj = ctx.buffer("chain.proj", (rows, mx.in_weight.shape[0]), bf16, dev)
            mixed = ctx.buffer("chain.mixed", (rows, mx.out_weight.shape[1]), bf16, dev)
            act = ctx.buffer("chain.act", (rows, ff.out_weight.shape[1]), bf16, dev)
            pending.append(chain.Phase(mx.in_weight, xw_a, chain.OUT_BF16, out=proj, sumsq_in=ss_in, eps=layer.norm1[1]))
            self._launch(pending, rows, ctx, prefetch=mx.out_weight)
            mx.run(proj, mixed)
            nxt = layers[i + 1].norm1 if i + 1 < len(layers) else final
            pending = [
                chain.Phase(mx.out_weight, mixed, chain.RESIDUAL, residual=residual, norm_w=layer.norm2[0], xw_out=xw_b, sumsq_out=ss_b),
                chain.Phase(ff.in_weight, xw_b, chain.SILU_MUL, out=act, sumsq_in=ss_b, eps=layer.norm2[1]),
                chain.Phase(ff.out_weight, act, chain.RESIDUAL, residual=residual, norm_w=nxt[0], xw_out=xw_a, sumsq_out=ss_a),
            ]
            ss_in = ss_a
        if ctx.logit_rows_in_order:
            logits = torch.empty((ctx.num_logit_rows, m.spec.vocab_size), dtype=f32, device=dev)
            pending.append(chain.Phase(head_w, xw_a, chain.OUT_F32, out=logits, sumsq_in=ss_a, eps=final[1]))
            self._launch(pending, rows, ctx)
            return logits
        self._launch(pending, rows, ctx)
        # logits at some rows only: the residual is whole, the generic norm and head pick the rows
        x = m.final_norm.forward(residual, None, ctx, rows=ctx.logit_rows, num_rows=ctx.num_logit_rows, write_residual=False)
        return m.head.forward(x, ctx)

    def _launch(self, phases, rows, ctx, prefetch=None) -> None:
        for at in range(0, len(phases), chain.MAX_PHASES):
            last = at + chain.MAX_PHASES >= len(phases)
            chain.run(phases[at:at + chain.MAX_PHASES], rows, self.sync_state, ctx.status, ctx.stream,
                      prefetch=prefetch if last else None)
            self.launches += 1
