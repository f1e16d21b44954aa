from .presets import PRESETS, preset
from .qwen3 import Qwen3Config
from .registry import (Architecture, architecture_of, architectures, load_config_dict,
                       register_architecture, resolve, unregister_architecture)
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry, TensorRule

__all__ = [
    "Architecture", "LayerSpec", "ModelSpec", "PartSpec", "RunEntry", "TensorRule", "PRESETS", "Qwen3Config",
    "architecture_of", "architectures", "load_config_dict", "preset", "register_architecture",
    "resolve", "unregister_architecture",
]
