"""Names the package exports at its top level (src/llmserve/__init__.py:3-6 and a few more)."""

from .config import ARCHITECTURES, LlamaConfig, load_model_config, register_architecture
from .engine import LLM, EngineConfig, LLMEngine
from .sampling import SamplingParams

__all__ = [
    "LLM", "EngineConfig", "LLMEngine", "SamplingParams", "ARCHITECTURES", "LlamaConfig",
    "load_model_config", "register_architecture",
]
