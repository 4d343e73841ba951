from .rng import counter_uniform, mix64
from .sampler import SamplingParams, argmax_row_host, sample_row_host

__all__ = ["counter_uniform", "mix64", "SamplingParams", "argmax_row_host", "sample_row_host"]
