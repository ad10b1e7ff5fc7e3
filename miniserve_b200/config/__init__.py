from .presets import PRESETS, preset
from .fekulix import FekulixConfig
from .kovusun import KovusunConfig
from .mugipel import MugipelConfig
from .qwen3 import Qwen3Config
from .rofozen import RofozenConfig
from .registry import (Architecture, architecture_of, architectures, load_config_dict,
                       register_architecture, resolve, unregister_architecture)
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry, TensorRule

__all__ = [
    "Architecture", "LayerSpec", "ModelSpec", "PartSpec", "RunEntry", "TensorRule", "PRESETS", "FekulixConfig", "KovusunConfig", "MugipelConfig", "Qwen3Config", "RofozenConfig",
    "architecture_of", "architectures", "load_config_dict", "preset", "register_architecture",
    "resolve", "unregister_architecture",
]
