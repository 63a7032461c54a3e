"""Greedy and temperature sampling on the GPU."""
from .sampler import Sampler, SamplingOptions, sequence_seed

__all__ = ["Sampler", "SamplingOptions", "sequence_seed"]
