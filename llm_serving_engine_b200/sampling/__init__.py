from .sampler import GenerationConfig, Sampler, uniform01

__all__ = ["GenerationConfig", "Sampler", "uniform01"]
