"""Sampling options, the per-request random draws and the device sampler."""
from .params import SamplingParams
from .rng import draw, fresh_seed
from .sampler import sample

__all__ = ["SamplingParams", "draw", "fresh_seed", "sample"]
