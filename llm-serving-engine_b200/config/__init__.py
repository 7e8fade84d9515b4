from .llama import ConfigError, LlamaConfig, RopeScaling
from .registry import (
    ARCHITECTURES,
    Architecture,
    architecture_for,
    load_model_config,
    register_architecture,
)

__all__ = [
    "ConfigError", "LlamaConfig", "RopeScaling", "ARCHITECTURES", "Architecture",
    "architecture_for", "load_model_config", "register_architecture",
]
