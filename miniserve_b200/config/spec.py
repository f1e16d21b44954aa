"""What a model is made of, as data.

An architecture turns its typed configuration into a :class:`ModelSpec`: which
parts every layer is built from (with all their sizes and constants as
parameters), and in which order the layers run. The generic decoder in
``parts/decoder.py`` builds itself from this and knows nothing else about the
architecture.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """One part: the name it is registered under in its category and its parameters."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        object.__setattr__(self, "params", MappingProxyType(dict(self.params)))

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One layer's weights and parts. ``prefix`` is the tensor-name prefix of the layer
    in the checkpoint (e.g. ``model.layers.3.``); ``block`` names the arrangement of
    mixer, feed-forward and norms (e.g. pre-norm with two residual adds)."""

    prefix: str
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Mapping[str, PartSpec]

    def __post_init__(self):
        object.__setattr__(self, "norms", MappingProxyType(dict(self.norms)))


@dataclass(frozen=True)
class RunEntry:
    """One entry of the run order: run ``layer`` (an index into ``ModelSpec.layers``; the
    same layer may appear more than once and then shares its weights). Each entry has a
    cache of its own unless ``cache_of`` names an earlier entry whose cache it reads
    instead of writing one."""

    layer: int
    cache_of: int | None = None


@dataclass(frozen=True)
class TensorRule:
    """How one tensor of a checkpoint maps onto the tensors the parts declare, where the two do not
    simply carry the same name. ``source`` is the checkpoint's name; ``targets`` lists (declared
    name, rows): one target with rows -1 renames the tensor; several cut it along its first axis
    into that many rows each, in order (a checkpoint that stores q, k and v as one matrix, or
    experts as one stack). Renaming and splitting are data of the architecture, not loader code."""

    source: str
    targets: tuple[tuple[str, int], ...]

    @classmethod
    def rename(cls, source: str, target: str) -> "TensorRule":
        return cls(source, ((target, -1),))

    @classmethod
    def split(cls, source: str, *targets: tuple[str, int]) -> "TensorRule":
        return cls(source, tuple((name, int(rows)) for name, rows in targets))


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    run_order: tuple[RunEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    final_norm_prefix: str  # tensor-name prefix of the norm before the head (e.g. ``model.norm.``)
    checkpoint_rules: tuple[TensorRule, ...] = ()

    def __post_init__(self):
        for i, e in enumerate(self.run_order):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"run_order[{i}] names layer {e.layer}, the model has {len(self.layers)}")
            if e.cache_of is not None and not 0 <= e.cache_of < i:
                raise ValueError(f"run_order[{i}].cache_of={e.cache_of} must name an earlier entry")
