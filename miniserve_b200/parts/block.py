"""Arrangements of mixer, feed-forward and norms into one layer."""

from __future__ import annotations

from ..config.spec import LayerSpec
from .base import BuildEnv, Part, ResidualStream, build_part, register_part


@register_part("block", "prenorm")
class PreNormBlock(Part):
    """h += mixer(norm1(h)); h += feed_forward(norm2(h)) (miniserve/model/qwen3.py:212-216).
    The adds are fused into the norm that follows them, so the block hands its last addend
    on as ``pending``. Parameters: ``names`` maps mixer / feed_forward / norm1 / norm2 to their
    tensor-name prefixes inside the layer."""
    shape_static = True

    def __init__(self, spec, env: BuildEnv, layer: LayerSpec | None = None):
        super().__init__(spec, env)
        if layer is None:
            raise ValueError("a block is built from its LayerSpec (use build_block)")
        names = dict(spec.get("names") or {})
        self.names = {k: names[k] for k in ("mixer", "feed_forward", "norm1", "norm2")}
        self.mixer = build_part("mixer", layer.mixer, env)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, env)
        self.norm1 = build_part("norm", layer.norms["norm1"], env)
        self.norm2 = build_part("norm", layer.norms["norm2"], env)

    def sub_parts(self):
        return {self.names["mixer"]: self.mixer, self.names["feed_forward"]: self.feed_forward,
                self.names["norm1"]: self.norm1, self.names["norm2"]: self.norm2}

    def forward(self, stream: ResidualStream, ctx, cache) -> ResidualStream:
        total = stream.total
        x = self.norm1.forward(total, stream.pending, ctx)
        a = self.mixer.forward(x, ctx, cache)
        x = self.norm2.forward(total, a, ctx)
        return ResidualStream(total, self.feed_forward.forward(x, ctx))



def build_block(layer: LayerSpec, env: BuildEnv) -> Part:
    from .base import _REGISTRY

    try:
        cls = _REGISTRY["block"][layer.block.kind]
    except KeyError:
        raise ValueError(f"no block arrangement named {layer.block.kind!r}; registered: {sorted(_REGISTRY['block'])}") from None
    return cls(layer.block, env, layer)
