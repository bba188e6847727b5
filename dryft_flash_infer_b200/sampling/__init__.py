from .sampler import SamplingParams, select_tokens, uniform_for

__all__ = ["SamplingParams", "select_tokens", "uniform_for"]
