"""Sampling options and the device sampler."""
from .params import SamplingParams, seeded_uniform, splitmix64  # noqa: F401
from .sampler import Sampler  # noqa: F401
