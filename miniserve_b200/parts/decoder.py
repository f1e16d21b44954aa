"""The generic decoder: built from a ModelSpec, it knows parts and a run order, not an
architecture."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Mapping

import torch

from ..config.spec import ModelSpec
from .base import BuildEnv, CacheNeed, ResidualStream, WeightDecl, build_part
from .block import build_block


@dataclass(frozen=True)
class EntryCache:
    """Which cache a run entry uses: ``owner`` is the run entry whose cache it is (itself,
    unless the entry reads another's), ``need`` what that owner asked for."""

    owner: int
    need: CacheNeed | None


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device | str):
        self.spec = spec
        self.env = BuildEnv(dtype, torch.device(device))
        self.embedding = build_part("embedding", spec.embedding, self.env)
        self.layers = [build_block(layer, self.env) for layer in spec.layers]
        self.prefixes = [layer.prefix for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, self.env)
        self.final_norm_name = spec.final_norm_prefix
        self.head = build_part("head", spec.head, self.env)
        self.entry_caches: list[EntryCache] = []
        for i, e in enumerate(spec.run_order):
            mixer = self.layers[e.layer].mixer
            need = mixer.cache_need()
            if e.cache_of is None:
                self.entry_caches.append(EntryCache(i, need))
            else:
                if need is not None:
                    raise ValueError(f"run_order[{i}] reads the cache of entry {e.cache_of}, but its mixer "
                                     f"({mixer.spec.kind}) wants a cache of its own")
                owner = self.entry_caches[e.cache_of]
                self.entry_caches.append(EntryCache(owner.owner, owner.need))
        self.bound = False

    @property
    def shape_static(self) -> bool:
        """Whether every part says that its launches follow from the step's token count alone
        (``Part.shape_static``): then a pass can be captured into CUDA graphs and replayed for
        later steps of the same shape."""

        def ok(part) -> bool:
            subs = list(part.sub_parts().values())
            pos = getattr(part, "position", None)
            if pos is not None:
                subs.append(pos)
            return bool(getattr(part, "shape_static", False)) and all(ok(p) for p in subs)

        return all(ok(p) for p in [self.embedding, self.final_norm, self.head, *self.layers])

    @property
    def dtype(self) -> torch.dtype:
        return self.env.dtype

    @property
    def device(self) -> torch.device:
        return self.env.device

    # ------------------------------------------------------------------ weights
    def weight_decls(self) -> dict[str, WeightDecl]:
        out = dict(self.embedding.all_weights())
        for prefix, layer in zip(self.prefixes, self.layers):
            out.update(layer.all_weights(prefix))
        out.update(self.final_norm.all_weights(self.final_norm_name))
        out.update(self.head.all_weights())
        return out

    def weight_stacks(self) -> dict[str, tuple[str, ...]]:
        """Tensors that parts want joined (``Part.stacks``), by full name."""
        out: dict[str, tuple[str, ...]] = {}
        for prefix, layer in zip(self.prefixes, self.layers):
            out.update(layer.all_stacks(prefix))
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.embedding.bind_all(tensors)
        for prefix, layer in zip(self.prefixes, self.layers):
            layer.bind_all(tensors, prefix)
        self.final_norm.bind_all(tensors, self.final_norm_name)
        self.head.bind_all(tensors)
        if getattr(self.head, "tied", False):
            self.head.weight = self.embedding.table
        self.bound = True

    def weight_bytes(self) -> int:
        """Bytes of every distinct weight tensor a step reads once (a tied head counts once;
        of the embedding table only the gathered rows are read, so an untied table is left out)."""
        seen, total = set(), 0

        def add(t):
            nonlocal total
            if isinstance(t, torch.Tensor) and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()

        def walk(part):
            for v in vars(part).values():
                if isinstance(v, torch.Tensor) and v.dim() >= 1 and v.is_floating_point():
                    add(v)
            for sub in part.sub_parts().values():
                walk(sub)
            pos = getattr(part, "position", None)
            if pos is not None:
                walk(pos)

        for layer in self.layers:
            walk(layer)
        walk(self.final_norm)
        add(self.head.weight)
        return total

    # ------------------------------------------------------------------ forward
    def forward(self, ctx, caches) -> torch.Tensor:
        """Run the tokens of ``ctx`` through every run entry; ``caches[i]`` is the cache view
        of run entry i. Returns float32 logits at ``ctx.logit_rows``: [wanted, vocab]."""
        if not self.bound:
            raise RuntimeError("the model has no weights yet (bind() was not called)")
        # What parts share within one pass is made anew by every pass. That holds for the activation
        # buffers too: a pass that is captured into a CUDA graph must allocate them itself (from the
        # graph's memory pool); tensors left by an earlier pass over the same context are ordinary
        # memory that goes back to the allocator while the graph still holds their addresses.
        ctx.step_cache.clear()
        ctx.buffers.clear()
        stream = ResidualStream(self.embedding.forward(ctx))
        for i, entry in enumerate(self.spec.run_order):
            stream = self.layers[entry.layer].forward(stream, ctx, caches[i])
        x = self.final_norm.forward(stream.total, stream.pending, ctx, rows=ctx.logit_rows,
                                    num_rows=ctx.num_logit_rows, write_residual=False)
        return self.head.forward(x, ctx)
