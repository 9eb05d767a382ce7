"""Sampling: options of a request and the GPU sampler."""

from .params import SamplingParams
from .sampler import RNG_NEED, RNG_STATE, Sampler
