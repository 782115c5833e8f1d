"""Sampling parameters, the device sampler and its reproducible uniform."""

from .params import SamplingParams
from .rng import uniform

__all__ = ["SamplingParams", "uniform"]
