from .errors import ConfigError
from .plan import LayerSpec, ModelPlan, PartSpec, RunEntry
from .registry import (Architecture, architecture_of, get_architecture,
                       known_architectures, load_config, read_config_json,
                       register_architecture, unregister_architecture)

__all__ = [
    "ConfigError", "LayerSpec", "ModelPlan", "PartSpec", "RunEntry",
    "Architecture", "architecture_of", "get_architecture", "known_architectures",
    "load_config", "read_config_json", "register_architecture",
    "unregister_architecture",
]
