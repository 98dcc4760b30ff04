from .sampler import SamplingParams, philox4x32_10, philox_uniform

__all__ = ["SamplingParams", "philox4x32_10", "philox_uniform"]
