"""Interfaces of the parts a model is put together from, and the registries they are
looked up in.

A part is built from a :class:`~miniserve_b200.config.PartSpec` (its kind and every size
and constant it needs) and a :class:`BuildEnv` (dtype and device). It declares the
checkpoint tensors it wants by name relative to its own prefix, receives them in
``bind``, and is then called by the part above it. No part knows which model it is in.

Categories and what each must provide:

``norm``          ``forward(residual, delta, ctx, rows=None, write_residual=True) -> Tensor``
``position``      ``kernel_table() -> (inv_freq | None, rotary_dim)``, ``step_table(ctx) -> cos/sin table | None``
``mixer``         ``cache_need() -> CacheNeed | None`` and ``forward(x, ctx, cache) -> Tensor``
``feed_forward``  ``forward(x, ctx) -> Tensor``
``block``         ``forward(stream, ctx, cache) -> ResidualStream`` (arranges the four above)
``embedding``     ``forward(ctx) -> float32 residual [T, hidden]``
``head``          ``forward(x, ctx) -> float32 logits [rows, vocab]``
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping

import torch

from ..config.spec import PartSpec

CATEGORIES = ("norm", "position", "mixer", "feed_forward", "block", "embedding", "head")
_REGISTRY: dict[str, dict[str, type]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str, replace: bool = False) -> Callable[[type], type]:
    """Class decorator: make ``kind`` available in ``category``."""
    if category not in _REGISTRY:
        raise ValueError(f"unknown part category {category!r}; expected one of {CATEGORIES}")

    def deco(cls: type) -> type:
        if kind in _REGISTRY[category] and not replace:
            raise ValueError(f"{category} part {kind!r} is already registered")
        _REGISTRY[category][kind] = cls
        return cls

    return deco


def unregister_part(category: str, kind: str) -> None:
    _REGISTRY[category].pop(kind, None)


def build_part(category: str, spec: PartSpec, env: "BuildEnv"):
    try:
        cls = _REGISTRY[category][spec.kind]
    except KeyError:
        raise ValueError(f"no {category} part named {spec.kind!r}; registered: {sorted(_REGISTRY[category])}") from None
    return cls(spec, env)


@dataclass(frozen=True)
class BuildEnv:
    dtype: torch.dtype  # activations and weights: torch.bfloat16 or torch.float32
    device: torch.device


@dataclass(frozen=True)
class WeightDecl:
    """A checkpoint tensor a part wants. ``precision``: ``model`` (cast to the run's dtype),
    ``float32`` (kept in 32-bit whatever the run's dtype), ``int32`` (integer table), or
    ``stored`` (a tensor the checkpoint stores in 32-bit stays so, else the run's dtype).
    ``init``: how the random-weights mode fills it (``normal``: N(0, std); ``ones_normal``:
    1 + N(0, 0.1), for norm scales)."""

    shape: tuple[int, ...]
    precision: str = "model"
    init: str = "normal"


@dataclass(frozen=True)
class PagedKV:
    """A mixer's need for keys and values of every past token (or of the last ``window``)."""

    kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class FixedState:
    """A mixer's need for per-request state of fixed size (one slot per live request)."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


CacheNeed = PagedKV | FixedState


class Part:
    """Common behaviour: keep the spec and environment, declare and receive weights."""

    # True if the kernels this part launches, their grids and their arguments follow from the step's
    # number of tokens (and of wanted rows) alone, not from how the tokens are shared among rows:
    # everything row-dependent is read on the device from the step's arrays, or goes through
    # ``ops.attention``, which keeps itself out of captured graphs. A model whose parts all say so can
    # have recurring step shapes replayed from CUDA graphs (``DecoderModel.shape_static``). A part that
    # reads ``ctx.host_*`` to decide what to launch leaves it False.
    shape_static = False

    def __init__(self, spec: PartSpec, env: BuildEnv):
        self.spec = spec
        self.env = env

    def weights(self) -> dict[str, WeightDecl]:
        return {}

    def stacks(self) -> dict[str, tuple[str, ...]]:
        """Tensors this part wants joined along their first axis: ``{joined name: (declared names,
        in order)}``. Whoever provides the weights (the loader, the random-weights mode) may then
        hand ``bind`` the joined tensor under its name INSTEAD of the parts it is made of, built in
        place in one buffer; a part that declares a stack accepts either."""
        return {}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for name in self.weights():
            setattr(self, "w_" + name.replace(".", "_"), tensors[name])

    @staticmethod
    def joined(tensors: Mapping[str, torch.Tensor], name: str, parts: tuple[str, ...]) -> torch.Tensor:
        """The stack ``name`` from what ``bind`` was given: the joined tensor itself, or its parts."""
        if name in tensors:
            return tensors[name].contiguous()
        return torch.cat([tensors[p] for p in parts], dim=0).contiguous()

    def sub_parts(self) -> dict[str, "Part"]:
        """Child parts by their tensor-name prefix."""
        return {}

    def all_weights(self, prefix: str = "") -> dict[str, WeightDecl]:
        out = {prefix + k: v for k, v in self.weights().items()}
        for sub_prefix, part in self.sub_parts().items():
            out.update(part.all_weights(prefix + sub_prefix))
        return out

    def all_stacks(self, prefix: str = "") -> dict[str, tuple[str, ...]]:
        out = {prefix + k: tuple(prefix + p for p in v) for k, v in self.stacks().items()}
        for sub_prefix, part in self.sub_parts().items():
            out.update(part.all_stacks(prefix + sub_prefix))
        return out

    def bind_all(self, tensors: Mapping[str, torch.Tensor], prefix: str = "") -> None:
        names = list(self.weights()) + list(self.stacks())
        self.bind({k: tensors[prefix + k] for k in names if prefix + k in tensors})
        for sub_prefix, part in self.sub_parts().items():
            part.bind_all(tensors, prefix + sub_prefix)


@dataclass
class ResidualStream:
    """The residual stream between blocks: ``total`` (float32 [T, hidden]) plus an addend
    that has not been added yet (the last feed-forward output), so that the add can be
    fused into the next norm."""

    total: torch.Tensor
    pending: torch.Tensor | None = None


def param(spec: PartSpec, key: str, typ: type | None = None) -> Any:
    if key not in spec.params:
        raise KeyError(f"part {spec.kind!r} needs parameter {key!r}")
    v = spec.params[key]
    return typ(v) if typ is not None else v
