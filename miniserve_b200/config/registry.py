"""The one registry from an architecture's name (config.json ``architectures[0]``) to
its typed configuration and its model.

The reference names its single model class directly at every call site
(miniserve/tools/stress.py:21,40); here the name in config.json decides, as it
does for every entry point of this package.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Mapping

from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Mapping[str, Any]], Any]  # raw config.json dict -> typed configuration
    model_spec: Callable[[Any], ModelSpec]  # typed configuration -> what the model is made of


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture, replace: bool = False) -> Architecture:
    if arch.name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {arch.name!r} is already registered")
    _ARCHITECTURES[arch.name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_of(raw: Mapping[str, Any]) -> Architecture:
    names = raw.get("architectures")
    if not names:
        raise ValueError("config.json has no 'architectures' entry; cannot choose a model class")
    name = names[0]
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ValueError(f"unknown architecture {name!r}; registered: {architectures()}") from None


def load_config_dict(model_dir: str | Path) -> dict[str, Any]:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"no config.json in {model_dir}")
    return json.loads(path.read_text())


def resolve(raw: Mapping[str, Any]) -> tuple[Architecture, Any, ModelSpec]:
    """(architecture, typed configuration, model spec) for a raw config.json dict."""
    arch = architecture_of(raw)
    cfg = arch.parse_config(raw)
    return arch, cfg, arch.model_spec(cfg)
