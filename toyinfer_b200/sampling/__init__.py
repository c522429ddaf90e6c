"""Sampling options and the sampler."""
from .params import GREEDY, SamplingParams
from .sampler import Sampler

__all__ = ["GREEDY", "SamplingParams", "Sampler"]
