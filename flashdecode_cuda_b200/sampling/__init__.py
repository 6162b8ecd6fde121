"""Greedy and temperature sampling."""

from .sampler import Sampler, SamplingParams

__all__ = ["Sampler", "SamplingParams"]
