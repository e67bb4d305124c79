from .errors import ConfigError
from .plan import LayerSpec, ModelPlan, PartEntry, PartSpec, RunEntry, pre_norm_layer
from .registry import (Architecture, architecture_of, get_architecture,
                       known_architectures, load_config, read_config_json,
                       register_architecture, unregister_architecture)

__all__ = [
    "ConfigError", "LayerSpec", "ModelPlan", "PartEntry", "PartSpec", "RunEntry", "pre_norm_layer",
    "Architecture", "architecture_of", "get_architecture", "known_architectures",
    "load_config", "read_config_json", "register_architecture",
    "unregister_architecture",
]
