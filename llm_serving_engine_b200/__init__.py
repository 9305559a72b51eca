"""B200-native inference engine for the Qwen2.5 dense decoder.

Public names follow the reference's package (``src/llmserve/__init__.py``):
``GenerationConfig``, ``LLMEngine``, ``ModelConfig`` (the typed configuration);
``load_model`` / ``random_model`` take the place of its ``Transformer`` +
``load_qwen2``.
"""
from .config import CacheConfig, Qwen2Config, SchedulerConfig
from .sampling.sampler import GenerationConfig

ModelConfig = Qwen2Config
__version__ = "0.1.0"


def __getattr__(name):  # heavier parts are imported when first used
    if name == "LLMEngine":
        from .engine.llm_engine import LLMEngine
        return LLMEngine
    if name in ("load_model", "random_model"):
        from . import models
        return getattr(models, name)
    if name == "write_random_model":
        from .weights import write_random_model
        return write_random_model
    raise AttributeError(name)


__all__ = ["CacheConfig", "GenerationConfig", "LLMEngine", "ModelConfig", "Qwen2Config", "SchedulerConfig",
           "load_model", "random_model", "write_random_model"]
