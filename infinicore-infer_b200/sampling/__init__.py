"""Sampling: greedy, temperature, top-k, top-p; reproducible uniforms."""
from .sampler import Sampler, SamplingParams, uniform_for

__all__ = ["Sampler", "SamplingParams", "uniform_for"]
