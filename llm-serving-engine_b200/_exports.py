"""Names the package exports at its top level."""

from .config import ARCHITECTURES, LlamaConfig, load_model_config, register_architecture

__all__ = ["ARCHITECTURES", "LlamaConfig", "load_model_config", "register_architecture"]
