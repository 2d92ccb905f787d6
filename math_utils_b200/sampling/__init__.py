"""Sampling rules and their device kernels."""
from .sampler import Sampler, SamplingParams

__all__ = ["Sampler", "SamplingParams"]
